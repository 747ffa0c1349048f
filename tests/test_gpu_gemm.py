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


@pytest.mark.parametrize("t", ALL_BLOCK_TYPES)
def test_gemm_every_format(gpu, oracle_mod, t):
    from saient_quartz_b200 import synth
    K, N, M = 2048, 130, 33
    w = synth.make_weights(t, K, N, tensor_id=711)
    X = synth.make_x(K, tensor_id=712, rows=M)
    for repack in (False, True):
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
