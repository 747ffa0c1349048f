"""quartz_b200: host-side mirror of the reference's CUDA wrapper over the C ABI.

The product is `libquartz_b200.so` (hand-written sm_100a CUDA behind the extern "C"
surface of include/quartz_b200.h).  This module loads it with ctypes and restates
the thin host types of the reference's src/cuda.rs -- GpuBuf (:59-90, 286-294),
GpuScratch (:94-128, 260-282), ensure_iq_grids (:131-140), verify_gemv_cuda
(:144-150), gpu_expert_slice (:242-258) -- with the same names and call order, so
tests and benchmarks exercise exactly what the Rust host would.  Nothing here
computes: there is no CPU fallback, and loading fails loudly when the library has
not been built.
"""
import ctypes as C
import os

import numpy as np

from . import build as _build
from . import synth  # noqa: F401  (re-exported)
from .synth import type_size as ggml_type_size

_HERE = os.path.dirname(os.path.abspath(__file__))
_lib = None

c_f32p = C.c_void_p
_SIGS = {
    # Part 1 (src/cuda.rs:6-55)
    "cuda_gemv": (None, [C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "cuda_set_iq3s_grid": (None, [C.c_void_p]),
    "cuda_set_iq2s_grid": (None, [C.c_void_p]),
    "cuda_set_iq2xxs_grid": (None, [C.c_void_p]),
    "cuda_set_iq2xs_grid": (None, [C.c_void_p]),
    "cuda_set_ksigns": (None, [C.c_void_p]),
    "cuda_mem_info": (None, [C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "cuda_alloc": (C.c_void_p, [C.c_size_t]),
    "cuda_drop": (None, [C.c_void_p]),
    "cuda_h2d": (None, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "cuda_d2h": (None, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "cuda_sync": (None, []),
    "cuda_vec_add": (None, [C.c_void_p, C.c_void_p, C.c_int]),
    "cuda_vec_scale_add": (None, [C.c_void_p, C.c_void_p, C.c_float, C.c_int]),
    "cuda_vec_zero": (None, [C.c_void_p, C.c_int]),
    "cuda_rms_norm": (None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]),
    "cuda_rope_yarn": (None, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float, C.c_int, C.c_int]),
    "cuda_kv_append": (None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "cuda_attn_score": (None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float]),
    "cuda_softmax_sink": (None, [C.c_void_p, C.c_int, C.c_float]),
    "cuda_attn_values": (None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int]),
    "cuda_swiglu": (None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]),
    "cuda_swiglu_oai": (None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]),
    "cuda_embed_lookup": (None, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_int, C.c_int]),
    "cuda_gemv_moe4": (None, [C.c_uint32] + [C.c_void_p] * 12 + [C.c_int, C.c_int, C.c_int]),
    "cuda_attn_score_all": (None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                   C.c_int, C.c_float]),
    "cuda_softmax_sink_all": (None, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "cuda_attn_values_all": (None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                    C.c_int]),
    # Part 2 (additions)
    "quartz_last_error": (C.c_int, []),
    "quartz_error_string": (C.c_char_p, []),
    "quartz_clear_error": (None, []),
    "quartz_set_stream": (None, [C.c_void_p]),
    "quartz_set_gemv_impl": (None, [C.c_int]),
    "quartz_launch_count": (C.c_longlong, []),
    "quartz_prefetch_next": (None, [C.c_void_p, C.c_size_t]),
    "cuda_set_iq3xxs_grid": (None, [C.c_void_p]),
    "cuda_repack_weights": (C.c_int, [C.c_uint32, C.c_void_p, C.c_int, C.c_int, C.c_int]),
    "cuda_unpack_weights": (C.c_int, [C.c_void_p]),
    "cuda_dequant": (None, [C.c_uint32, C.c_void_p, C.c_void_p, C.c_int, C.c_longlong]),
    "cuda_quantize_x": (None, [C.c_void_p, C.c_int, C.c_int]),
    "cuda_rms_norm_q": (None, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "cuda_swiglu_q": (None, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]),
    "cuda_gemv_q_supported": (C.c_int, [C.c_uint32, C.c_void_p, C.c_int]),
    "cuda_gemv_q": (None, [C.c_uint32, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]),
    "cuda_rope_kv": (None, [C.c_void_p] * 5 + [C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float, C.c_int,
                            C.c_int]),
    "cuda_attn_decode": (None, [C.c_void_p] * 4 + [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float,
                                C.c_void_p, C.c_int]),
    "quartz_set_pdl": (None, [C.c_int]),
    "quartz_graph_begin": (C.c_int, []),
    "quartz_graph_end": (C.c_void_p, []),
    "quartz_graph_launch": (None, [C.c_void_p]),
    "quartz_graph_destroy": (None, [C.c_void_p]),
    "cuda_gemv_noalloc": (None, [C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "cuda_gemm": (None, [C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]),
    "cuda_gemm_bf16": (None, [C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]),
    "cuda_gemv_rmsnorm": (None, [C.c_uint32, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]),
    "cuda_gemv_swiglu": (None, [C.c_uint32, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                C.c_int]),
    "cuda_h2d_async": (None, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "cuda_d2h_async": (None, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "cuda_host_alloc": (C.c_void_p, [C.c_size_t]),
    "cuda_host_free": (None, [C.c_void_p]),
    "cuda_gemv_chain_supported": (C.c_int, [C.c_int, C.c_void_p]),
    "cuda_gemv_chain": (None, [C.c_int, C.c_void_p]),
    "cuda_gemv_batch": (None, [C.c_int, C.c_void_p]),
    "cuda_attn_block": (None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                               C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_float, C.c_float, C.c_int, C.c_int, C.c_int]),
    "cuda_step_set": (None, [C.c_void_p, C.c_int, C.c_int]),
    "cuda_step_rope_table": (None, [C.c_void_p, C.c_int, C.c_float, C.c_float, C.c_int]),
    "cuda_embed_lookup_dev": (None, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_int]),
    "cuda_attn_step_supported": (C.c_int, [C.c_int, C.c_int, C.c_int]),
    "cuda_attn_step": (None, [C.c_void_p] * 6 + [C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int,
                              C.c_float, C.c_void_p, C.c_float, C.c_float, C.c_int, C.c_int, C.c_int]),
    "cuda_moe_ffn_dev": (None, [C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int]),
    "cuda_embed_lookup_rows": (None, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_int, C.c_int]),
    "cuda_rms_norm_rows": (None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "cuda_rope_kv_rows": (None, [C.c_void_p] * 5 + [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float, C.c_int, C.c_int]),
    "cuda_attn_prompt": (None, [C.c_void_p] * 4 + [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_void_p]),
    "cuda_gemv_experts": (None, [C.c_uint32, C.c_void_p, C.c_size_t, C.c_void_p, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p,
                                 C.c_int, C.c_int]),
    "cuda_moe_decode_act": (None, [C.c_void_p] * 6 + [C.c_int, C.c_int, C.c_int]),
    "cuda_moe_decode_combine": (None, [C.c_void_p] * 5 + [C.c_int, C.c_int, C.c_int]),
    "cuda_router_topk": (None, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "cuda_moe_ffn": (None, [C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                            C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int]),
    "quartz_nccl_id_bytes": (C.c_size_t, []),
    "quartz_nccl_unique_id": (C.c_int, [C.c_void_p]),
    "quartz_nccl_init": (C.c_int, [C.c_int, C.c_int, C.c_void_p]),
    "quartz_mgpu_allgather": (None, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "quartz_nccl_shutdown": (None, []),
    "quartz_mgpu_handle_bytes": (C.c_size_t, []),
    "quartz_set_device": (C.c_int, [C.c_int]),
    "quartz_mgpu_init": (C.c_int, [C.c_int, C.c_int, C.c_size_t, C.c_void_p]),
    "quartz_mgpu_attach": (C.c_int, [C.c_void_p]),
    "quartz_mgpu_data": (C.c_void_p, []),
    "cuda_gemv_push": (None, [C.c_uint32, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int]),
    "cuda_gemv_batch_push": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p]),
    "quartz_mgpu_wait_in_next_push": (None, []),
    "cuda_gemm_push": (C.c_int, [C.c_uint32, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_size_t, C.c_size_t]),
    "cuda_gemv_chain_push": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "cuda_push_rows": (None, [C.c_void_p, C.c_int, C.c_int, C.c_size_t, C.c_size_t]),
    "quartz_mgpu_wait": (None, []),
    "quartz_mgpu_fuse_next_wait": (None, []),
    "quartz_mgpu_shutdown": (None, []),
}

# The 28 symbols the reference's Rust host binds (src/cuda.rs:6-55).
REFERENCE_SYMBOLS = [
    "cuda_gemv", "cuda_set_iq3s_grid", "cuda_set_iq2s_grid", "cuda_set_iq2xxs_grid", "cuda_set_iq2xs_grid",
    "cuda_set_ksigns", "cuda_mem_info", "cuda_alloc", "cuda_drop", "cuda_h2d", "cuda_d2h", "cuda_sync",
    "cuda_vec_add", "cuda_vec_scale_add", "cuda_vec_zero", "cuda_rms_norm", "cuda_rope_yarn", "cuda_kv_append",
    "cuda_attn_score", "cuda_softmax_sink", "cuda_attn_values", "cuda_swiglu", "cuda_swiglu_oai",
    "cuda_embed_lookup", "cuda_gemv_moe4", "cuda_attn_score_all", "cuda_softmax_sink_all", "cuda_attn_values_all",
]


def library_path():
    return _build.LIB


def lib():
    """The loaded C-ABI library.  Raises if it was not built: there is no fallback path."""
    global _lib
    if _lib is None:
        path = library_path()
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} is missing: build it first (python __graft_entry__.py or "
                f"python saient-quartz_b200/build.py); quartz_b200 has no CPU fallback")
        L = C.CDLL(path)
        for name, (res, args) in _SIGS.items():
            fn = getattr(L, name)   # AttributeError = the library does not export a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


class ChainOp(C.Structure):
    """qz_chain_op of include/quartz_b200.h."""
    _fields_ = [("ggml_type", C.c_uint32), ("n_mats", C.c_int), ("d_w", C.POINTER(C.c_void_p)),
                ("d_y", C.POINTER(C.c_void_p)), ("in_dim", C.c_int), ("out_dim", C.c_int), ("accumulate", C.c_int),
                ("src_mode", C.c_int), ("d_a", C.c_void_p), ("d_b", C.c_void_p), ("oai", C.c_int)]


def chain_op(ggml_type, w_ptrs, y_ptrs, in_dim, out_dim, accumulate, src_mode, a_ptr, b_ptr=None, oai=0):
    """Build one ChainOp; the pointer arrays are kept alive on the returned object."""
    n = len(w_ptrs)
    W = (C.c_void_p * n)(*w_ptrs)
    Y = (C.c_void_p * n)(*y_ptrs)
    op = ChainOp(ggml_type, n, C.cast(W, C.POINTER(C.c_void_p)), C.cast(Y, C.POINTER(C.c_void_p)), in_dim, out_dim,
                 1 if accumulate else 0, src_mode, a_ptr, b_ptr, oai)
    op._keep = (W, Y)
    return op


def declared_symbols():
    """Every symbol include/quartz_b200.h declares (parsed from the header)."""
    import re
    hdr = open(os.path.join(_HERE, "..", "include", "quartz_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    return sorted(set(re.findall(r"\b((?:cuda|quartz)_[a-z0-9_]+)\s*\(", hdr)))


def check_error(what=""):
    L = lib()
    code = L.quartz_last_error()
    if code != 0:
        msg = L.quartz_error_string().decode()
        L.quartz_clear_error()
        raise RuntimeError(f"quartz_b200 error {code} {what}: {msg}")


# ---------------------------------------------------------------------------------------
# Host mirror of src/cuda.rs
# ---------------------------------------------------------------------------------------
class GpuBuf:
    """Owns one cuda_alloc'ed device buffer (src/cuda.rs:59-90)."""

    def __init__(self, ptr, nbytes):
        self.ptr = ptr
        self.bytes = nbytes

    @classmethod
    def upload(cls, data):
        data = np.ascontiguousarray(data)
        nbytes = data.nbytes
        ptr = lib().cuda_alloc(max(nbytes, 1))
        if not ptr:
            raise MemoryError(f"cudaMalloc failed for {nbytes} bytes")
        if nbytes:
            lib().cuda_h2d(ptr, data.ctypes.data, nbytes)
        return cls(ptr, nbytes)

    @classmethod
    def alloc_f32(cls, n):
        ptr = lib().cuda_alloc(max(4 * n, 4))
        if not ptr:
            raise MemoryError(f"cudaMalloc failed for {n} f32s")
        return cls(ptr, 4 * n)

    upload_f32 = upload

    def download(self, dtype=np.float32, count=None, offset_bytes=0):
        item = np.dtype(dtype).itemsize
        if count is None:
            count = (self.bytes - offset_bytes) // item
        out = np.empty(count, dtype=dtype)
        if count:
            lib().cuda_d2h(out.ctypes.data, self.ptr + offset_bytes, count * item)
        lib().cuda_sync()
        return out

    def drop(self):
        if self.ptr:
            lib().cuda_drop(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.drop()
        except Exception:
            pass


class GpuSlice:
    """A view into an uploaded 3-D expert tensor (src/cuda.rs:242-258)."""

    def __init__(self, ptr, ggml_type):
        self.ptr = ptr
        self.ggml_type = ggml_type


def gpu_expert_slice(buf, ggml_type, expert, n_elems_per_expert):
    return GpuSlice(buf.ptr + expert * ggml_type_size(ggml_type, n_elems_per_expert), ggml_type)


class GpuScratch:
    """d_x / d_y reused by every gemv call: H2D x, cuda_gemv, D2H y, sync (src/cuda.rs:94-128)."""

    def __init__(self, max_in, max_out):
        self.max_in, self.max_out = max_in, max_out
        self.d_x = GpuBuf.alloc_f32(max_in)
        self.d_y = GpuBuf.alloc_f32(max_out)

    def _run(self, x, ptr, ggml_type, in_dim, out_dim):
        x = np.ascontiguousarray(x, dtype=np.float32)
        # the reference does not check these (src/main.rs:646-666 overruns d_x); this mirror does
        if x.size > self.max_in or out_dim > self.max_out:
            raise ValueError("GpuScratch: vector larger than the scratch buffers")
        L = lib()
        L.cuda_h2d(self.d_x.ptr, x.ctypes.data, x.nbytes)
        L.cuda_gemv(ggml_type, ptr, self.d_x.ptr, self.d_y.ptr, in_dim, out_dim)
        out = np.empty(out_dim, dtype=np.float32)
        L.cuda_d2h(out.ctypes.data, self.d_y.ptr, out_dim * 4)
        L.cuda_sync()
        return out

    def gemv(self, x, data, ggml_type, in_dim, out_dim):
        return self._run(x, data.ptr, ggml_type, in_dim, out_dim)

    def gemv_slice(self, x, slc, in_dim, out_dim):
        return self._run(x, slc.ptr, slc.ggml_type, in_dim, out_dim)


_grids_done = False


def ensure_iq_grids():
    """Upload the IQ codebooks once per process (src/cuda.rs:131-140), IQ3_XXS included."""
    global _grids_done
    if _grids_done:
        return
    from .iq_tables import load_tables
    t = load_tables()
    L = lib()
    L.cuda_set_iq3s_grid(t["iq3s"].ctypes.data)
    L.cuda_set_iq2s_grid(t["iq2s"].ctypes.data)
    L.cuda_set_iq2xxs_grid(t["iq2xxs"].ctypes.data)
    L.cuda_set_iq2xs_grid(t["iq2xs"].ctypes.data)
    L.cuda_set_ksigns(t["ksigns"].ctypes.data)
    L.cuda_set_iq3xxs_grid(t["iq3xxs"].ctypes.data)
    _grids_done = True


def verify_gemv_cuda(x, data, ggml_type, in_dim, out_dim, repack=False):
    """Run cuda_gemv on a freshly uploaded raw tensor (src/cuda.rs:144-150)."""
    ensure_iq_grids()
    buf = GpuBuf.upload(data)
    if repack:
        lib().cuda_repack_weights(ggml_type, buf.ptr, in_dim, out_dim, 1)
    sc = GpuScratch(in_dim, out_dim)
    y = sc.gemv(x, buf, ggml_type, in_dim, out_dim)
    check_error("verify_gemv_cuda")
    return y


def dequant_cuda(data, ggml_type, in_dim, n_rows, repack=False):
    """cuda_dequant on a freshly uploaded tensor; returns f32 [n_rows * in_dim]."""
    ensure_iq_grids()
    buf = GpuBuf.upload(data)
    if repack:
        lib().cuda_repack_weights(ggml_type, buf.ptr, in_dim, n_rows, 1)
    out = GpuBuf.alloc_f32(in_dim * n_rows)
    lib().cuda_dequant(ggml_type, buf.ptr, out.ptr, in_dim, n_rows)
    res = out.download()
    check_error("dequant_cuda")
    return res
