"""ctypes front-end of the CPU oracle -- TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke check and the CPU-baseline leg of bench.py import this
module.  It wraps oracle/libquartz_oracle.so (the C restatement of the
reference's src/dequant.rs) and, where present, oracle/_ref/libkernels_ref.so
(the reference's own CUDA kernels, used on a GPU box as an A/B baseline and a
secondary result check).
"""
import ctypes as C
import os

import numpy as np

from . import build as _build

_lib = None
_tables = None


def lib():
    global _lib
    if _lib is None:
        path = _build.ORACLE_SO
        if not os.path.exists(path):
            path = _build.build_oracle()
        L = C.CDLL(path)
        L.qz_type_size.restype = C.c_size_t
        L.qz_type_size.argtypes = [C.c_uint32, C.c_size_t]
        L.qz_f16_to_f32.restype = C.c_float
        L.qz_f16_to_f32.argtypes = [C.c_uint16]
        L.qz_ksigns.restype = C.POINTER(C.c_uint8)
        L.qz_max_threads.restype = C.c_int
        for name in ("qz_set_iq2xxs_grid", "qz_set_iq2xs_grid", "qz_set_iq2s_grid", "qz_set_iq3s_grid",
                     "qz_set_iq3xxs_grid"):
            getattr(L, name).argtypes = [C.c_void_p]
            getattr(L, name).restype = None
        L.qz_dequant.argtypes = [C.c_void_p, C.c_uint32, C.c_size_t, C.c_void_p]
        L.qz_gemv.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_size_t, C.c_size_t, C.c_void_p, C.c_int]
        L.qz_gemm.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_size_t, C.c_size_t, C.c_size_t,
                              C.c_void_p, C.c_int]
        L.qz_row_norms.argtypes = [C.c_void_p, C.c_uint32, C.c_size_t, C.c_size_t, C.c_void_p, C.c_int]
        L.qz_gemv_f64.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_size_t, C.c_size_t, C.c_void_p,
                                  C.c_int]
        _lib = L
    return _lib


def set_tables(tables):
    """Hand the IQ codebooks (dict from the host package's iq_tables.load_tables) to the oracle."""
    global _tables
    L = lib()
    _tables = {k: np.ascontiguousarray(v) for k, v in tables.items()}  # keep alive
    L.qz_set_iq2xxs_grid(_tables["iq2xxs"].ctypes.data)
    L.qz_set_iq2xs_grid(_tables["iq2xs"].ctypes.data)
    L.qz_set_iq2s_grid(_tables["iq2s"].ctypes.data)
    L.qz_set_iq3s_grid(_tables["iq3s"].ctypes.data)
    L.qz_set_iq3xxs_grid(_tables["iq3xxs"].ctypes.data)


def ksigns():
    return np.ctypeslib.as_array(lib().qz_ksigns(), shape=(128,)).copy()


def max_threads():
    return lib().qz_max_threads()


def _u8(a):
    a = np.ascontiguousarray(a)
    return a.view(np.uint8).reshape(-1)


def dequant(data, ggml_type, n_elems):
    data = _u8(data)
    out = np.empty(n_elems, dtype=np.float32)
    rc = lib().qz_dequant(data.ctypes.data, ggml_type, n_elems, out.ctypes.data)
    if rc != 0:
        raise ValueError(f"dequant: unsupported ggml_type {ggml_type}")
    return out


def gemv(x, data, ggml_type, in_dim, out_dim, threads=0):
    x = np.ascontiguousarray(x, dtype=np.float32)
    data = _u8(data)
    y = np.empty(out_dim, dtype=np.float32)
    rc = lib().qz_gemv(x.ctypes.data, data.ctypes.data, ggml_type, in_dim, out_dim, y.ctypes.data, threads)
    if rc != 0:
        raise ValueError(f"gemv: unsupported ggml_type {ggml_type}")
    return y


def gemm(x, data, ggml_type, in_dim, out_dim, n, threads=0):
    x = np.ascontiguousarray(x, dtype=np.float32)
    data = _u8(data)
    out = np.empty((n, out_dim), dtype=np.float32)
    rc = lib().qz_gemm(x.ctypes.data, data.ctypes.data, ggml_type, in_dim, out_dim, n, out.ctypes.data,
                       threads)
    if rc != 0:
        raise ValueError(f"gemm: unsupported ggml_type {ggml_type}")
    return out


def row_norms(data, ggml_type, in_dim, out_dim, threads=0):
    data = _u8(data)
    out = np.empty(out_dim, dtype=np.float64)
    rc = lib().qz_row_norms(data.ctypes.data, ggml_type, in_dim, out_dim, out.ctypes.data, threads)
    if rc != 0:
        raise ValueError(f"row_norms: unsupported ggml_type {ggml_type}")
    return out


def gemv_f64(x, data, ggml_type, in_dim, out_dim, threads=0):
    x = np.ascontiguousarray(x, dtype=np.float32)
    data = _u8(data)
    y = np.empty(out_dim, dtype=np.float64)
    rc = lib().qz_gemv_f64(x.ctypes.data, data.ctypes.data, ggml_type, in_dim, out_dim, y.ctypes.data,
                           threads)
    if rc != 0:
        raise ValueError(f"gemv_f64: unsupported ggml_type {ggml_type}")
    return y


def tolerance(data, ggml_type, in_dim, out_dim, x):
    """Per-row bound 1e-3 * ||w_row||_2 * ||x||_2 (the acceptance bound for GEMV/GEMM outputs)."""
    xn = float(np.linalg.norm(np.asarray(x, dtype=np.float64)))
    return 1e-3 * row_norms(data, ggml_type, in_dim, out_dim) * xn


def ref_kernels():
    """The reference's own CUDA kernels (oracle/_ref), or None when not built."""
    path = _build.REF_SO
    if not os.path.exists(path):
        return None
    L = C.CDLL(path)
    L.cuda_gemv.argtypes = [C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
    L.cuda_gemv.restype = None
    for name in ("cuda_set_iq3s_grid", "cuda_set_iq2s_grid", "cuda_set_iq2xxs_grid", "cuda_set_iq2xs_grid",
                 "cuda_set_ksigns"):
        getattr(L, name).argtypes = [C.c_void_p]
        getattr(L, name).restype = None
    L.cuda_sync.restype = None
    return L
