"""cuda_gemv_noalloc: the GEMV entry point for hosts that cannot allocate device memory at call
time (inside a stream capture, under a fixed memory plan, or when another allocator owns the
device).  Its activation scratch is an array built into the library, so this file checks, through
the C ABI, that two calls in a row reproduce cuda_gemv, that free device memory does not move
between them, and that a problem larger than the built-in scratch is refused with a clear error.
Collected last on purpose: a failure here cannot hide the results of the other GPU tests."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _free_bytes(L):
    f, t = ctypes.c_size_t(0), ctypes.c_size_t(0)
    L.cuda_mem_info(ctypes.byref(f), ctypes.byref(t))
    return f.value


@pytest.mark.parametrize("t,K,N", [(12, 4096, 1000), (14, 4096, 515), (8, 2048, 333), (13, 512, 40)])
def test_noalloc_matches_cuda_gemv_twice(gpu, oracle_mod, t, K, N):
    from saient_quartz_b200 import synth
    L = gpu.lib()
    w = synth.make_weights(t, K, N, tensor_id=301)
    dw = gpu.GpuBuf.upload(w)
    L.cuda_repack_weights(t, dw.ptr, K, N, 1)
    dx, dy, dy_ref = gpu.GpuBuf.alloc_f32(K), gpu.GpuBuf.alloc_f32(N), gpu.GpuBuf.alloc_f32(N)
    free_after_first = None
    for call in range(2):                      # two calls in a row share the built-in scratch
        x = synth.make_x(K, tensor_id=310 + call)
        L.cuda_h2d(dx.ptr, x.ctypes.data, x.nbytes)
        L.cuda_gemv(t, dw.ptr, dx.ptr, dy_ref.ptr, K, N)
        L.cuda_vec_zero(dy.ptr, N)
        L.cuda_gemv_noalloc(t, dw.ptr, dx.ptr, dy.ptr, K, N)
        y, y_ref = dy.download(), dy_ref.download()
        gpu.check_error("cuda_gemv_noalloc")
        tol = oracle_mod.tolerance(w, t, K, N, x)          # 1e-3 * ||w_row|| * ||x||, as everywhere
        assert np.all(np.abs(y.astype(np.float64) - y_ref) <= tol)
        assert np.all(np.abs(y.astype(np.float64) - oracle_mod.gemv(x, w, t, K, N)) <= tol)
        if call == 0:
            free_after_first = _free_bytes(L)
        else:
            assert _free_bytes(L) == free_after_first       # the second call took no device memory


def test_noalloc_rejects_sizes_beyond_its_scratch(gpu):
    L = gpu.lib()
    K, N = 65536, 2                                        # 65536 > the 32768 the built-in scratch holds
    dw = gpu.GpuBuf.upload(np.zeros(K // 256 * 144 * N, np.uint8))
    dx = gpu.GpuBuf.upload(np.ones(K, np.float32))
    dy = gpu.GpuBuf.upload(np.full(N, 7.0, np.float32))
    L.cuda_gemv_noalloc(12, dw.ptr, dx.ptr, dy.ptr, K, N)
    assert L.quartz_last_error() == 5                       # QZ_ERR_TOO_LARGE
    assert b"32768" in L.quartz_error_string()
    L.quartz_clear_error()
    assert np.all(dy.download() == 7.0)                     # output untouched
