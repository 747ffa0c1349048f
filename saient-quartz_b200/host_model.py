"""ctypes front-end of libquartz_host.so: the C++ restatement of the reference's GpuWeights /
GpuForwardState (src/cuda.rs:154-236, 301-851), plus the Llama-3-8B-shaped synthetic model of the
decode benchmark."""
import ctypes as C
import os

import numpy as np

from . import build as _build
from . import synth

_host = None


class QhConfig(C.Structure):
    _fields_ = [(n, C.c_int) for n in (
        "vocab_size", "embed_dim", "n_heads", "n_kv_heads", "n_layers", "ffn_dim", "head_dim", "n_experts",
        "n_experts_used", "moe_renorm", "clamped_swiglu", "swa_window", "rope_neox", "yarn_orig_ctx", "max_seq")] + [
        ("rope_theta", C.c_float), ("yarn_scale", C.c_float)]


ROLES = {n: i for i, n in enumerate([
    "EMBED", "LM_HEAD", "FINAL_NORM", "Q", "K", "V", "O", "GATE", "UP", "DOWN", "ATTN_NORM", "FFN_NORM", "Q_NORM",
    "K_NORM", "Q_BIAS", "K_BIAS", "V_BIAS", "O_BIAS", "SINKS", "MOE_GATE", "MOE_UP", "MOE_DOWN", "ROUTER_W",
    "ROUTER_B", "MOE_GATE_BIAS", "MOE_UP_BIAS", "MOE_DOWN_BIAS"])}


def host_lib():
    global _host
    if _host is None:
        from . import lib
        lib()   # the CUDA library first (the host library links against it)
        path = _build.HOST_LIB
        if not os.path.exists(path):
            raise RuntimeError(f"{path} is missing: run the build first")
        H = C.CDLL(path)
        H.qh_create.restype = C.c_void_p
        H.qh_create.argtypes = [C.POINTER(QhConfig)]
        H.qh_destroy.argtypes = [C.c_void_p]
        H.qh_set_tensor.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_uint32, C.c_void_p, C.c_size_t, C.c_int]
        H.qh_finalize.argtypes = [C.c_void_p]
        H.qh_set_kv.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int]
        H.qh_forward_step.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
        H.qh_forward_step_fused.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
        H.qh_forward_step_chained.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
        H.qh_step_device.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int]
        H.qh_read_hidden.argtypes = [C.c_void_p, C.c_void_p]
        H.qh_launches_last_step.restype = C.c_longlong
        H.qh_launches_last_step.argtypes = [C.c_void_p]
        H.qh_graphs_recorded.argtypes = [C.c_void_p]
        H.qh_force_host_router.argtypes = [C.c_int]
        H.qh_prefill.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        H.qh_get_kv.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        _host = H
    return _host


# Llama-3-8B architecture in the project's fixed "Q4_K_M" layout: attn q/k/v/o and ffn gate/up in
# Q4_K, ffn down and the output head in Q6_K, token embedding in Q4_K.
LLAMA3_8B = dict(vocab_size=128256, embed_dim=4096, n_heads=32, n_kv_heads=8, n_layers=32, ffn_dim=14336,
                 head_dim=128, rope_theta=500000.0, max_seq=2048)
Q4K_M_TYPES = dict(Q=12, K=12, V=12, O=12, GATE=12, UP=12, DOWN=14, LM_HEAD=14, EMBED=12)


class HostModel:
    """A model resident on the GPU, driven through the C++ host mirror."""

    def __init__(self, repack=True, types=Q4K_M_TYPES, seed=synth.DEFAULT_SEED, keep_host=False, **cfg):
        from . import ensure_iq_grids
        ensure_iq_grids()
        self.H = host_lib()
        full = dict(n_experts=0, n_experts_used=0, moe_renorm=1, clamped_swiglu=0, swa_window=0, rope_neox=0,
                    yarn_orig_ctx=0, yarn_scale=1.0)
        full.update(cfg)
        self.cfg = full
        self.c = QhConfig(**{k: (float(v) if k in ("rope_theta", "yarn_scale") else int(v)) for k, v in full.items()})
        self.m = self.H.qh_create(C.byref(self.c))
        if not self.m:
            raise RuntimeError("qh_create failed")
        self.types = dict(types)
        self.host = {} if keep_host else None
        self.repack = repack
        self.seed = seed
        self.weight_bytes = 0

    @classmethod
    def from_gguf(cls, path, max_seq=0, repack=True):
        """Load a model from a GGUF file through qh_load_gguf (configuration and tensor names as the reference
        reads them, src/main.rs:96-215, 357-414)."""
        from . import ensure_iq_grids
        ensure_iq_grids()
        self = cls.__new__(cls)
        self.H = host_lib()
        self.H.qh_load_gguf.restype = C.c_void_p
        self.H.qh_load_gguf.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_void_p]
        self.H.qh_load_error.restype = C.c_char_p
        self.c = QhConfig()
        self.m = self.H.qh_load_gguf(str(path).encode(), max_seq, int(repack), C.byref(self.c))
        if not self.m:
            raise RuntimeError("qh_load_gguf failed: " + self.H.qh_load_error().decode())
        self.cfg = {name: getattr(self.c, name) for name, _ in QhConfig._fields_}
        self.host, self.repack, self.types, self.weight_bytes = None, repack, None, 0
        return self

    def set(self, role, layer, ggml_type, arr):
        arr = np.ascontiguousarray(arr)
        rc = self.H.qh_set_tensor(self.m, ROLES[role], layer, ggml_type, arr.ctypes.data, arr.nbytes, int(self.repack))
        if rc != 0:
            raise RuntimeError(f"qh_set_tensor({role}, layer {layer}) failed: {rc}")
        if self.host is not None:
            self.host[(role, layer)] = (ggml_type, arr)

    def fill_synthetic(self):
        """Seeded random-init weights of the architecture (norm weights ~ 1 + 0.1 N(0,1))."""
        c, t = self.cfg, self.types
        d, fd, q_d = c["embed_dim"], c["ffn_dim"], c["n_heads"] * c["head_dim"]
        kv_d = c["n_kv_heads"] * c["head_dim"]
        rng = np.random.Generator(np.random.PCG64([self.seed, 0xC0F]))
        tid = 1000

        def w(role, layer, K, N):
            nonlocal tid
            tid += 1
            a = synth.make_weights(t[role], K, N, seed=self.seed, tensor_id=tid)
            self.set(role, layer, t[role], a)
            if role != "EMBED":
                self.weight_bytes += a.nbytes

        def norm(role, layer, n):
            self.set(role, layer, 0, (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32))

        w("EMBED", 0, d, c["vocab_size"])
        for l in range(c["n_layers"]):
            w("Q", l, d, q_d); w("K", l, d, kv_d); w("V", l, d, kv_d); w("O", l, q_d, d)
            w("GATE", l, d, fd); w("UP", l, d, fd); w("DOWN", l, fd, d)
            norm("ATTN_NORM", l, d); norm("FFN_NORM", l, d)
        norm("FINAL_NORM", 0, d)
        w("LM_HEAD", 0, d, c["vocab_size"])
        self.finalize()

    def finalize(self):
        rc = self.H.qh_finalize(self.m)
        if rc != 0:
            raise RuntimeError(f"qh_finalize failed: {rc}")

    def fill_kv(self, n_pos, keep=False):
        """f32 KV cache pre-filled with N(0,1) for positions 0..n_pos-1."""
        kv_d = self.cfg["n_kv_heads"] * self.cfg["head_dim"]
        out = []
        for l in range(self.cfg["n_layers"]):
            rng = np.random.Generator(np.random.PCG64([self.seed, 0xCAC4E, l]))
            k = rng.standard_normal((n_pos, kv_d), dtype=np.float32)
            v = rng.standard_normal((n_pos, kv_d), dtype=np.float32)
            self.H.qh_set_kv(self.m, l, k.ctypes.data, v.ctypes.data, n_pos)
            if keep:
                out.append((k, v))
        return out

    def read_kv(self, layer, pos0, n_pos):
        """Rows [pos0, pos0 + n_pos) of a layer's K and V caches."""
        kv_d = self.cfg["n_kv_heads"] * self.cfg["head_dim"]
        k, v = np.empty((n_pos, kv_d), np.float32), np.empty((n_pos, kv_d), np.float32)
        if self.H.qh_get_kv(self.m, layer, k.ctypes.data, v.ctypes.data, pos0, n_pos) != 0:
            raise RuntimeError("qh_get_kv failed")
        return k, v

    def prefill(self, tokens, pos0=0, want_logits=True):
        """Batched prefill of a prompt (qh_prefill); returns the last token's logits."""
        tok = np.ascontiguousarray(tokens, dtype=np.int32)
        logits = np.empty(self.cfg["vocab_size"], dtype=np.float32) if want_logits else None
        rc = self.H.qh_prefill(self.m, tok.ctypes.data, int(tok.size), int(pos0), logits.ctypes.data if want_logits else None)
        if rc != 0:
            from . import lib
            raise RuntimeError(f"prefill failed: {rc} ({lib().quartz_error_string().decode()})")
        return logits

    def step(self, token, pos, fused=False):
        logits = np.empty(self.cfg["vocab_size"], dtype=np.float32)
        fn = (self.H.qh_forward_step_chained if fused == 2 else self.H.qh_forward_step_fused) if fused else self.H.qh_forward_step
        rc = fn(self.m, token, pos, 1, logits.ctypes.data)
        if rc != 0:
            from . import lib
            raise RuntimeError(f"forward step failed: {rc} ({lib().quartz_error_string().decode()})")
        return logits

    def step_device(self, token, pos, fused=False):
        return self.H.qh_step_device(self.m, token, pos, int(fused))

    def hidden(self):
        h = np.empty(self.cfg["embed_dim"], dtype=np.float32)
        self.H.qh_read_hidden(self.m, h.ctypes.data)
        return h

    def launches(self):
        return int(self.H.qh_launches_last_step(self.m))

    def graphs_recorded(self):
        """How many times a step sequence has been recorded into a graph for this model."""
        return int(self.H.qh_graphs_recorded(self.m))

    def close(self):
        if self.m:
            self.H.qh_destroy(self.m)
            self.m = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
