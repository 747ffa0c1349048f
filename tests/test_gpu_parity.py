"""GPU parity: the CUDA path, called through the C ABI, against the CPU oracle.

Bars: dequantized weights bit-exact (u32 compare); GEMV outputs within
max_j |y_j - ref_j| <= 1e-3 * ||w_j||_2 * ||x||_2 (the stated acceptance bound), and
for information the tighter max|d| / max|y| that the reference's own --verify-gemv
mode uses (src/main.rs:2653-2659, threshold 1e-3)."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "dequant_golden.npz")
ALL_TYPES = [0, 1, 30, 2, 3, 6, 7, 8, 20, 10, 12, 13, 14, 16, 17, 18, 21, 22]
STREAM_TYPES = [12, 14, 8, 2, 3, 6, 7, 16, 17, 22, 18, 21, 13, 10, 20]


# Regression bound, close to what is measured: the streaming kernels carry x in 16-bit block-fixed-point form
# (worst case 8.7e-5 * ||w|| * ||x||, measured 1e-6 .. 5e-5 for N(0,1) activations) and sum in f32; the acceptance
# bound (1e-3) would let a wrong sub-block scale or a dropped 32-run through, this one does not.
REGRESSION = 1e-4


def _check_gemv(oracle_mod, y, x, w, t, K, N, verify_bar=1e-3, regression=None):
    ref = oracle_mod.gemv(x, w, t, K, N)
    tol = oracle_mod.tolerance(w, t, K, N, x)
    err = np.abs(y.astype(np.float64) - ref.astype(np.float64))
    assert np.all(np.isfinite(y))
    assert np.all(err <= tol), f"type {t} {K}->{N}: max err/tol {np.max(err / np.maximum(tol, 1e-30)):.3g}"
    if regression is not None:   # tol = 1e-3 * ||w_j|| * ||x||
        assert np.all(err <= regression * 1e3 * tol), \
            f"type {t} {K}->{N}: max err / (||w|| ||x||) = {np.max(err / np.maximum(1e3 * tol, 1e-30)):.3g}"
    if N >= 64:   # the reference's --verify-gemv metric
        assert err.max() / max(np.abs(ref).max(), 1e-30) < verify_bar
    return float(np.max(err / np.maximum(tol, 1e-30)))


def test_dequant_bit_exact_golden(gpu, oracle_mod):
    g = np.load(GOLDEN)
    from saient_quartz_b200 import synth
    K, N = 512, 6
    for t in ALL_TYPES:
        name = synth.FORMATS[t][0]
        got = gpu.dequant_cuda(g[f"w_{name}"], t, K, N)
        assert np.array_equal(got.view(np.uint32), g[f"deq_{name}"].view(np.uint32)), name


@pytest.mark.parametrize("t", ALL_TYPES)
def test_dequant_bit_exact_seeded_raw_and_planes(gpu, oracle_mod, t):
    from saient_quartz_b200 import synth
    K, N = 2048, 33
    w = synth.make_weights(t, K, N, tensor_id=21)
    want = oracle_mod.dequant(w, t, K * N)
    got = gpu.dequant_cuda(w, t, K, N)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    got2 = gpu.dequant_cuda(w, t, K, N, repack=True)   # plane layout where the format has one
    assert np.array_equal(got2.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("t", [14, 8])
def test_repack_round_trip_restores_bytes(gpu, t):
    from saient_quartz_b200 import synth
    K, N = 2048, 19
    w = synth.make_weights(t, K, N, tensor_id=22)
    buf = gpu.GpuBuf.upload(w)
    L = gpu.lib()
    assert L.cuda_repack_weights(t, buf.ptr, K, N, 1) == 1
    packed = buf.download(np.uint8)
    assert not np.array_equal(packed, w) and np.array_equal(np.sort(packed), np.sort(w))
    assert L.cuda_repack_weights(t, buf.ptr, K, N, 1) == 0      # already repacked: refused
    assert L.quartz_last_error() != 0
    L.quartz_clear_error()
    assert L.cuda_unpack_weights(buf.ptr) == 1
    assert np.array_equal(buf.download(np.uint8), w)
    assert L.cuda_unpack_weights(buf.ptr) == 0
    gpu.check_error()


def test_repack_declined_when_planes_would_be_misaligned(gpu):
    from saient_quartz_b200 import synth
    K, N = 1024, 8    # 4 blocks per row: not a multiple of 8
    w = synth.make_weights(14, K, N)
    buf = gpu.GpuBuf.upload(w)
    assert gpu.lib().cuda_repack_weights(14, buf.ptr, K, N, 1) == 0
    assert np.array_equal(buf.download(np.uint8), w)
    assert gpu.lib().cuda_repack_weights(12, buf.ptr, 1024, 8, 1) == 0   # Q4_K streams from raw
    gpu.check_error()


@pytest.mark.parametrize("t", ALL_TYPES)
def test_gemv_golden_small(gpu, oracle_mod, t):
    from saient_quartz_b200 import synth
    g = np.load(GOLDEN)
    name = synth.FORMATS[t][0]
    K, N = 512, 6
    y = gpu.verify_gemv_cuda(g["x"], g[f"w_{name}"], t, K, N)
    _check_gemv(oracle_mod, y, g["x"], g[f"w_{name}"], t, K, N)
    tol = oracle_mod.tolerance(g[f"w_{name}"], t, K, N, g["x"])
    assert np.all(np.abs(y - g[f"y64_{name}"]) <= tol)


@pytest.mark.parametrize("t", ALL_TYPES)
@pytest.mark.parametrize("shape", [(4096, 512), (2048, 37), (1024, 1), (256, 5), (6144, 130)])
def test_gemv_seeded_shapes(gpu, oracle_mod, t, shape):
    """Ragged out_dim, a single row, one block per row, and K with 96 units per row."""
    from saient_quartz_b200 import synth
    K, N = shape
    w = synth.make_weights(t, K, N, tensor_id=31)
    x = synth.make_x(K, tensor_id=32)
    for repack in (False, True):
        y = gpu.verify_gemv_cuda(x, w, t, K, N, repack=repack)
        _check_gemv(oracle_mod, y, x, w, t, K, N)


@pytest.mark.parametrize("t", [2, 3, 6, 7, 8, 20])
def test_gemv_k_not_multiple_of_64(gpu, oracle_mod, t):
    from saient_quartz_b200 import synth
    K, N = 96, 9
    w = synth.make_weights(t, K, N, tensor_id=33)
    x = synth.make_x(K, tensor_id=34)
    y = gpu.verify_gemv_cuda(x, w, t, K, N)
    _check_gemv(oracle_mod, y, x, w, t, K, N)


def test_config0_q4k_4096x4096(gpu, oracle_mod):
    """The reference-runnable configuration: one Q4_K GEMV, 4096 -> 4096, batch 1."""
    from saient_quartz_b200 import synth
    K = N = 4096
    w = synth.make_weights(12, K, N)
    x = synth.make_x(K)
    y = gpu.verify_gemv_cuda(x, w, 12, K, N)
    r = _check_gemv(oracle_mod, y, x, w, 12, K, N)
    assert r < 0.05   # far inside the bound: x carries 16-bit block-fixed-point precision


@pytest.mark.parametrize("label,t,K,N", [
    ("k/v", 12, 4096, 1024), ("gate/up", 12, 4096, 14336), ("down", 14, 14336, 4096),
    ("q8_0", 8, 4096, 4096), ("70B gate shard", 12, 8192, 3584), ("70B down shard", 14, 28672, 1024)])
def test_config1_and_sharded_shapes(gpu, oracle_mod, label, t, K, N):
    from saient_quartz_b200 import synth
    w = synth.make_weights(t, K, N, tensor_id=41)
    x = synth.make_x(K, tensor_id=42)
    y = gpu.verify_gemv_cuda(x, w, t, K, N, repack=True)
    _check_gemv(oracle_mod, y, x, w, t, K, N, regression=REGRESSION)


@pytest.mark.parametrize("t,K,N", [(12, 8192, 28672), (14, 28672, 8192)])
def test_70b_shaped_matrices_full_size(gpu, oracle_mod, t, K, N):
    """The two Llama-3-70B-shaped FFN matrices of the row-sharded benchmark, whole, on one GPU."""
    from saient_quartz_b200 import synth
    w = synth.make_weights(t, K, N, tensor_id=45)
    x = synth.make_x(K, tensor_id=46)
    y = gpu.verify_gemv_cuda(x, w, t, K, N, repack=True)
    _check_gemv(oracle_mod, y, x, w, t, K, N, regression=REGRESSION)


def _adversarial_activations(K):
    """Activation vectors that stress the 16-bit block-fixed-point form the streaming kernels convert x into
    (one scale per run of 32 values): name -> vector."""
    r = np.random.Generator(np.random.PCG64([0xAD7]))
    out = {}
    x = (1e-2 * r.standard_normal(K)).astype(np.float32)
    x[37] = 1e4
    x[K - 5] = -3e3
    out["one large outlier inside a run of small values"] = x
    x = r.standard_normal(K).astype(np.float32)
    x[64:192] *= np.float32(1e-20)
    x[1024:1056] *= np.float32(1e-36)      # a run below the flush threshold next to ordinary runs
    out["runs of very different magnitude, one of them tiny"] = x
    out["whole vector tiny"] = (1e-25 * r.standard_normal(K)).astype(np.float32)
    x = np.full(K, 3.25, np.float32)
    x[1::2] = -3.25
    out["every element at the run maximum, alternating sign"] = x
    x = np.zeros(K, np.float32)
    x[100] = 1.0
    out["a single non-zero element"] = x
    x = r.standard_normal(K).astype(np.float32)
    x[::32] = 127.49 * np.abs(x).max()      # the maximum of every run sits at its first element
    out["run maxima that all round to the top code"] = x
    return out


@pytest.mark.parametrize("t", [12, 14, 8, 7, 17])
def test_gemv_adversarial_activations(gpu, oracle_mod, t):
    """The acceptance bound must hold for any finite activation vector, not only for N(0,1) draws: the
    block-fixed-point conversion bounds its own error by 8.7e-5 * ||w|| * ||x|| (Cauchy-Schwarz over the
    per-run rounding errors), 11 times inside the bound.  Runs whose maximum is below 2^-110 are taken as
    zero (their products underflow in f32 as well)."""
    from saient_quartz_b200 import synth
    K, N = 4096, 192
    w = synth.make_weights(t, K, N, tensor_id=47)
    for name, x in _adversarial_activations(K).items():
        for repack in (True, False):
            y = gpu.verify_gemv_cuda(x, w, t, K, N, repack=repack)
            ref = oracle_mod.gemv(x, w, t, K, N)
            tol = oracle_mod.tolerance(w, t, K, N, x)
            err = np.abs(y.astype(np.float64) - ref.astype(np.float64))
            assert np.all(np.isfinite(y)), name
            assert np.all(err <= np.maximum(tol, 1e-37)), f"type {t}, {name}: max err/tol {np.max(err / np.maximum(tol, 1e-37)):.3g}"


@pytest.mark.parametrize("t", [12, 14, 8])
def test_gemv_non_finite_activations_propagate(gpu, oracle_mod, t):
    """A NaN or an infinity anywhere in x makes every output non-finite, as in the f32 reference (where
    x_k * w_k is NaN or +-inf and poisons the row sum)."""
    from saient_quartz_b200 import synth
    K, N = 4096, 64
    w = synth.make_weights(t, K, N, tensor_id=48)
    for bad in (np.nan, np.inf, -np.inf):
        x = synth.make_x(K, tensor_id=49).copy()
        x[777] = bad
        y = gpu.verify_gemv_cuda(x, w, t, K, N, repack=True)
        with np.errstate(all="ignore"):
            ref = oracle_mod.gemv(x, w, t, K, N)
        assert not np.any(np.isfinite(ref))
        assert not np.any(np.isfinite(y)), bad


def test_lm_head_full_size(gpu, oracle_mod):
    """Q6_K 4096 -> 128256 (431 MB), full comparison against the oracle."""
    from saient_quartz_b200 import synth
    K, N = 4096, 128256
    w = synth.make_weights(14, K, N, tensor_id=43)
    x = synth.make_x(K, tensor_id=44)
    y = gpu.verify_gemv_cuda(x, w, 14, K, N, repack=True)
    _check_gemv(oracle_mod, y, x, w, 14, K, N, regression=REGRESSION)


@pytest.mark.parametrize("t", STREAM_TYPES)
def test_both_streaming_kernels_agree(gpu, oracle_mod, t):
    """The TMA-staged ring and the register-streaming kernel share the per-unit integer arithmetic;
    only the order of the final f32 row sums differs."""
    from saient_quartz_b200 import synth
    L = gpu.lib()
    try:
        for (K, N) in [(4096, 1030), (14336, 257), (1024, 64), (8192, 100), (28672, 33)]:
            w = synth.make_weights(t, K, N, tensor_id=55)
            x = synth.make_x(K, tensor_id=56)
            L.quartz_set_gemv_impl(0)
            y_tma = gpu.verify_gemv_cuda(x, w, t, K, N, repack=True)
            L.quartz_set_gemv_impl(1)
            y_ldg = gpu.verify_gemv_cuda(x, w, t, K, N, repack=True)
            _check_gemv(oracle_mod, y_tma, x, w, t, K, N, regression=REGRESSION)
            _check_gemv(oracle_mod, y_ldg, x, w, t, K, N, regression=REGRESSION)
            tol = oracle_mod.tolerance(w, t, K, N, x)
            assert np.all(np.abs(y_tma - y_ldg) <= 1e-2 * tol), (t, K, N)
    finally:
        L.quartz_set_gemv_impl(0)


@pytest.mark.parametrize("t", STREAM_TYPES)
def test_gemv_linearity_and_zero(gpu, t):
    """Size-independent properties: W*0 = 0 exactly; W*(2x) = 2*(W*x) exactly (power-of-two scaling
    commutes with the block-fixed-point activation format and with every f32 rounding)."""
    from saient_quartz_b200 import synth
    K, N = 4096, 1024
    w = synth.make_weights(t, K, N, tensor_id=51)
    x = synth.make_x(K, tensor_id=52)
    y1 = gpu.verify_gemv_cuda(x, w, t, K, N, repack=True)
    y2 = gpu.verify_gemv_cuda(2.0 * x, w, t, K, N, repack=True)
    y0 = gpu.verify_gemv_cuda(np.zeros(K, np.float32), w, t, K, N, repack=True)
    assert np.array_equal(y2, 2.0 * y1)
    assert np.all(y0 == 0.0)


@pytest.mark.parametrize("t", [12, 14, 7, 17])
def test_gemv_moe4(gpu, oracle_mod, t):
    """cuda_gemv_moe4 (src/cuda.rs:39-45): expert slices of one 3-D tensor, shared and distinct x."""
    from saient_quartz_b200 import synth
    K, N, E = 2048, 96, 6
    w = synth.make_weights(t, K, N * E, tensor_id=61)
    buf = gpu.GpuBuf.upload(w)
    L = gpu.lib()
    L.cuda_repack_weights(t, buf.ptr, K, N, E)
    per = synth.type_size(t, K * N)
    experts = [4, 0, 5, 2]
    xs = [synth.make_x(K, tensor_id=70 + i) for i in range(4)]
    for shared in (True, False):
        dx = [gpu.GpuBuf.upload(xs[0] if shared else xs[i]) for i in range(4)]
        dy = gpu.GpuBuf.alloc_f32(4 * N)
        for n_act in (4, 2):
            L.cuda_vec_zero(dy.ptr, 4 * N)
            sl = [gpu.gpu_expert_slice(buf, t, e, K * N).ptr for e in experts]
            L.cuda_gemv_moe4(t, sl[0], sl[1], sl[2], sl[3], dx[0].ptr, dx[1].ptr, dx[2].ptr, dx[3].ptr,
                             dy.ptr, dy.ptr + 4 * N, dy.ptr + 8 * N, dy.ptr + 12 * N, n_act, K, N)
            y = dy.download().reshape(4, N)
            gpu.check_error()
            for i in range(4):
                if i < n_act:
                    we = w[experts[i] * per:(experts[i] + 1) * per]
                    _check_gemv(oracle_mod, y[i], xs[0] if shared else xs[i], we, t, K, N)
                else:
                    assert np.all(y[i] == 0.0)   # slots >= n_act untouched


def test_unknown_type_zero_fills_and_reports(gpu):
    """src/cuda_kernels.cu:1073-1077: zero y, stderr line; plus the sticky status."""
    L = gpu.lib()
    dy = gpu.GpuBuf.upload(np.ones(64, np.float32))
    dx = gpu.GpuBuf.upload(np.ones(256, np.float32))
    dw = gpu.GpuBuf.upload(np.zeros(1024, np.uint8))
    L.cuda_gemv(15, dw.ptr, dx.ptr, dy.ptr, 256, 64)
    assert np.all(dy.download() == 0.0)
    assert L.quartz_last_error() == 1
    L.quartz_clear_error()
    L.cuda_gemv(12, dw.ptr, dx.ptr, dy.ptr, 100, 4)     # in_dim not a multiple of 256
    assert L.quartz_last_error() == 2
    L.quartz_clear_error()
    L.cuda_gemv(12, dw.ptr, dx.ptr, dy.ptr, 256, 0)     # empty output: nothing to do
    assert L.quartz_last_error() == 0


def test_embed_lookup_all_types(gpu, oracle_mod):
    from saient_quartz_b200 import synth
    D, V = 512, 11
    L = gpu.lib()
    for t in ALL_TYPES:
        w = synth.make_weights(t, D, V, tensor_id=81)
        buf = gpu.GpuBuf.upload(w)
        out = gpu.GpuBuf.alloc_f32(D)
        L.cuda_embed_lookup(out.ptr, buf.ptr, t, 7, D)
        want = oracle_mod.dequant(w, t, D * V).reshape(V, D)[7]
        assert np.array_equal(out.download().view(np.uint32), want.view(np.uint32)), t
    gpu.check_error()


def test_against_reference_cuda_kernels(gpu, oracle_mod, tables):
    """Secondary check and oracle pin: the reference's own kernels (oracle/_ref, compiled
    unmodified from its src/cuda_kernels.cu) agree with the oracle and with this library."""
    R = oracle_mod.ref_kernels()
    if R is None:
        pytest.skip("oracle/_ref not built (reference tree was not mounted at build time)")
    from saient_quartz_b200 import synth
    R.cuda_set_iq3s_grid(tables["iq3s"].ctypes.data)
    R.cuda_set_iq2s_grid(tables["iq2s"].ctypes.data)
    R.cuda_set_iq2xxs_grid(tables["iq2xxs"].ctypes.data)
    R.cuda_set_iq2xs_grid(tables["iq2xs"].ctypes.data)
    R.cuda_set_ksigns(tables["ksigns"].ctypes.data)
    K, N = 4096, 256
    for t in [0, 1, 30, 6, 7, 8, 10, 12, 13, 14, 16, 17, 20, 21, 22]:
        w = synth.make_weights(t, K, N, tensor_id=91)
        x = synth.make_x(K, tensor_id=92)
        dw, dx, dy = gpu.GpuBuf.upload(w), gpu.GpuBuf.upload(x), gpu.GpuBuf.alloc_f32(N)
        R.cuda_gemv(t, dw.ptr, dx.ptr, dy.ptr, K, N)
        R.cuda_sync()
        y_ref_gpu = dy.download()
        _check_gemv(oracle_mod, y_ref_gpu, x, w, t, K, N)         # reference GPU vs oracle
        y = gpu.verify_gemv_cuda(x, w, t, K, N, repack=True)
        tol = oracle_mod.tolerance(w, t, K, N, x)
        assert np.all(np.abs(y - y_ref_gpu) <= tol), t          # this library vs reference GPU


def test_embed_lookup_bit_exact_against_reference_kernel(gpu, oracle_mod):
    """The reference's own cuda_embed_lookup (src/cuda_kernels.cu:701-750, 1172-1186; Q5_1, IQ4_NL and BF16 rows)
    dequantizes on the GPU with the CPU path's formulas: its rows, this library's cuda_embed_lookup /
    cuda_dequant and the oracle must agree bit for bit (u32 compare) -- a pin of the oracle by the reference
    itself."""
    import ctypes as C
    R = oracle_mod.ref_kernels()
    if R is None:
        pytest.skip("oracle/_ref not built (reference tree was not mounted at build time)")
    from saient_quartz_b200 import synth
    R.cuda_embed_lookup.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_int, C.c_int]
    R.cuda_embed_lookup.restype = None
    L = gpu.lib()
    D, V = 1024, 9
    for t in (7, 20, 30):
        w = synth.make_weights(t, D, V, tensor_id=95)
        buf = gpu.GpuBuf.upload(w)
        o_ref, o_me = gpu.GpuBuf.alloc_f32(D), gpu.GpuBuf.alloc_f32(D)
        want = oracle_mod.dequant(w, t, D * V).reshape(V, D)
        for token in (0, 4, V - 1):
            R.cuda_embed_lookup(o_ref.ptr, buf.ptr, t, token, D)
            R.cuda_sync()
            L.cuda_embed_lookup(o_me.ptr, buf.ptr, t, token, D)
            a, b = o_ref.download().view(np.uint32), o_me.download().view(np.uint32)
            assert np.array_equal(a, want[token].view(np.uint32)), (t, token, "reference kernel vs oracle")
            assert np.array_equal(a, b), (t, token, "reference kernel vs this library")
    gpu.check_error()
