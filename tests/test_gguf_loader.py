"""GGUF reader / device loader (saient-quartz_b200/host/gguf_loader.cpp, the counterpart of
src/gguf.rs:53-123) against files written with the gguf package: header, metadata accessors, tensor
table, data section alignment, byte-exact tensor contents; malformed files are refused.  The GPU
part uploads tensors through the staging buffers + repack hook and runs cuda_gemv on them."""
import ctypes as C
import os

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _host_lib(pkg):
    from saient_quartz_b200 import build
    path = build.build_host()
    L = C.CDLL(path)
    L.qg_open.restype = C.c_void_p
    L.qg_open.argtypes = [C.c_char_p]
    L.qg_close.argtypes = [C.c_void_p]
    L.qg_last_error.restype = C.c_char_p
    for name, res, args in [("qg_version", C.c_uint32, [C.c_void_p]), ("qg_data_offset", C.c_uint64, [C.c_void_p]),
                            ("qg_n_tensors", C.c_int, [C.c_void_p]), ("qg_find_tensor", C.c_int, [C.c_void_p, C.c_char_p]),
                            ("qg_tensor_name", C.c_char_p, [C.c_void_p, C.c_int]),
                            ("qg_tensor_type", C.c_uint32, [C.c_void_p, C.c_int]),
                            ("qg_tensor_n_dims", C.c_int, [C.c_void_p, C.c_int]),
                            ("qg_tensor_dim", C.c_uint64, [C.c_void_p, C.c_int, C.c_int]),
                            ("qg_tensor_bytes", C.c_uint64, [C.c_void_p, C.c_int]),
                            ("qg_tensor_data", C.c_void_p, [C.c_void_p, C.c_int]),
                            ("qg_meta_u32", C.c_int, [C.c_void_p, C.c_char_p, C.c_void_p]),
                            ("qg_meta_u64", C.c_int, [C.c_void_p, C.c_char_p, C.c_void_p]),
                            ("qg_meta_f32", C.c_int, [C.c_void_p, C.c_char_p, C.c_void_p]),
                            ("qg_meta_str", C.c_char_p, [C.c_void_p, C.c_char_p]),
                            ("qg_meta_array_len", C.c_int, [C.c_void_p, C.c_char_p, C.c_void_p]),
                            ("qg_upload_tensor", C.c_void_p, [C.c_void_p, C.c_int, C.c_int, C.c_void_p])]:
        getattr(L, name).restype = res
        getattr(L, name).argtypes = args
    return L


def _write_fixture(path, alignment=None):
    """A small llama-shaped file: metadata of several value types, an f32 norm, a Q4_K and a Q6_K matrix, an
    IQ2_XS 3-D expert tensor.  Returns {name: (ggml_type, dims (fastest first), raw bytes)}."""
    import gguf
    from saient_quartz_b200 import synth
    w = gguf.GGUFWriter(path, "llama")
    if alignment:
        w.add_custom_alignment(alignment)
    w.add_uint32("llama.block_count", 3)
    w.add_uint32("llama.embedding_length", 512)
    w.add_float32("llama.rope.freq_base", 500000.0)
    w.add_uint64("test.big", 1 << 40)
    w.add_string("general.name", "fixture")
    w.add_array("tokenizer.ggml.tokens", ["<s>", "a", "bc"])
    w.add_array("tokenizer.ggml.token_type", [1, 2, 3, 4])
    want = {}
    norm = (1.0 + 0.01 * np.arange(512)).astype(np.float32)
    w.add_tensor("blk.0.attn_norm.weight", norm)
    want["blk.0.attn_norm.weight"] = (0, [512], norm.tobytes())
    for tid, (name, t, K, N) in enumerate((("blk.0.attn_q.weight", 12, 512, 256), ("blk.0.ffn_down.weight", 14, 2048, 96))):
        raw = synth.make_weights(t, K, N, tensor_id=40 + tid)
        rb = synth.type_size(t, K)
        w.add_tensor(name, raw.reshape(N, rb), raw_dtype=gguf.GGMLQuantizationType(t))
        want[name] = (t, [K, N], raw.tobytes())
    E, K, N = 4, 256, 64
    raw = np.concatenate([synth.make_weights(17, K, N, tensor_id=50 + e) for e in range(E)])
    w.add_tensor("blk.0.ffn_gate_exps.weight", raw.reshape(E, N, synth.type_size(17, K)), raw_dtype=gguf.GGMLQuantizationType(17))
    want["blk.0.ffn_gate_exps.weight"] = (17, [K, N, E], raw.tobytes())
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return want


@pytest.mark.parametrize("alignment", [None, 64])
def test_reader_matches_what_was_written(pkg, tmp_path, alignment):
    import gguf
    L = _host_lib(pkg)
    path = str(tmp_path / "fixture.gguf")
    want = _write_fixture(path, alignment)
    f = L.qg_open(path.encode())
    assert f, L.qg_last_error()
    assert L.qg_version(f) == 3
    assert L.qg_n_tensors(f) == len(want)
    assert L.qg_data_offset(f) % (alignment or 32) == 0
    rd = gguf.GGUFReader(path)
    assert L.qg_data_offset(f) == rd.data_offset
    u32, u64, f32 = C.c_uint32(), C.c_uint64(), C.c_float()
    assert L.qg_meta_u32(f, b"llama.block_count", C.byref(u32)) == 1 and u32.value == 3
    assert L.qg_meta_u64(f, b"llama.embedding_length", C.byref(u64)) == 1 and u64.value == 512   # u32 widens
    assert L.qg_meta_u64(f, b"test.big", C.byref(u64)) == 1 and u64.value == 1 << 40
    assert L.qg_meta_u32(f, b"test.big", C.byref(u32)) == 0                                      # u64 does not narrow
    assert L.qg_meta_f32(f, b"llama.rope.freq_base", C.byref(f32)) == 1 and f32.value == 500000.0
    assert L.qg_meta_str(f, b"general.architecture") == b"llama"
    assert L.qg_meta_str(f, b"general.name") == b"fixture"
    assert L.qg_meta_str(f, b"llama.block_count") is None and L.qg_meta_str(f, b"absent") is None
    assert L.qg_meta_array_len(f, b"tokenizer.ggml.tokens", C.byref(u64)) == 1 and u64.value == 3
    assert L.qg_meta_array_len(f, b"tokenizer.ggml.token_type", C.byref(u64)) == 1 and u64.value == 4
    for name, (t, dims, raw) in want.items():
        i = L.qg_find_tensor(f, name.encode())
        assert i >= 0 and L.qg_tensor_name(f, i) == name.encode()
        assert L.qg_tensor_type(f, i) == t
        assert L.qg_tensor_n_dims(f, i) == len(dims)
        assert [L.qg_tensor_dim(f, i, d) for d in range(len(dims))] == dims
        assert L.qg_tensor_bytes(f, i) == len(raw)
        got = C.string_at(L.qg_tensor_data(f, i), len(raw))
        assert got == raw, name
    assert L.qg_find_tensor(f, b"nope") == -1
    L.qg_close(f)


def test_malformed_files_are_refused(pkg, tmp_path):
    L = _host_lib(pkg)
    path = str(tmp_path / "fixture.gguf")
    _write_fixture(path)
    blob = open(path, "rb").read()
    cases = {"magic": b"GGUX" + blob[4:], "version": blob[:4] + (9).to_bytes(4, "little") + blob[8:],
             "truncated_meta": blob[:60], "tiny": blob[:8]}
    for label, data in cases.items():
        p = str(tmp_path / (label + ".gguf"))
        open(p, "wb").write(data)
        assert not L.qg_open(p.encode()), label
        assert L.qg_last_error(), label
    # a table that points past the end of the file: the file opens, the tensor has no data
    p = str(tmp_path / "short.gguf")
    open(p, "wb").write(blob[:len(blob) - 4096])
    f = L.qg_open(p.encode())
    assert f
    last = L.qg_n_tensors(f) - 1
    assert L.qg_tensor_data(f, last) is None
    L.qg_close(f)
    assert not L.qg_open(str(tmp_path / "missing.gguf").encode())


@pytest.mark.gpu
def test_upload_and_gemv(gpu, oracle_mod, tmp_path):
    from saient_quartz_b200 import synth
    L = _host_lib(gpu)
    Q = gpu.lib()
    path = str(tmp_path / "fixture.gguf")
    want = _write_fixture(path)
    f = L.qg_open(path.encode())
    assert f
    for name in ("blk.0.attn_q.weight", "blk.0.ffn_down.weight"):
        t, (K, N), raw = want[name]
        rep = C.c_int(-1)
        dev = L.qg_upload_tensor(f, L.qg_find_tensor(f, name.encode()), 1, C.byref(rep))
        assert dev, L.qg_last_error()
        assert rep.value in (0, 1)
        x = synth.make_x(K, tensor_id=3).reshape(-1)
        dx, dy = gpu.GpuBuf.upload(x), gpu.GpuBuf.alloc_f32(N)
        Q.cuda_gemv(t, dev, dx.ptr, dy.ptr, K, N)
        y = dy.download()
        gpu.check_error(name)
        w = np.frombuffer(raw, dtype=np.uint8)
        ref = oracle_mod.gemv(x, w, t, K, N)
        tol = oracle_mod.tolerance(w, t, K, N, x)
        assert np.all(np.abs(y - ref) <= tol), name
        Q.cuda_drop(dev)
    # the 3-D expert tensor: expert 2 through its byte offset (src/cuda.rs:250-257)
    t, (K, N, E), raw = want["blk.0.ffn_gate_exps.weight"]
    dev = L.qg_upload_tensor(f, L.qg_find_tensor(f, b"blk.0.ffn_gate_exps.weight"), 1, None)
    assert dev
    one = synth.type_size(t, K * N)
    x = synth.make_x(K, tensor_id=4).reshape(-1)
    dx, dy = gpu.GpuBuf.upload(x), gpu.GpuBuf.alloc_f32(N)
    Q.cuda_gemv(t, dev + 2 * one, dx.ptr, dy.ptr, K, N)
    w = np.frombuffer(raw, dtype=np.uint8)[2 * one:3 * one]
    assert np.all(np.abs(dy.download() - oracle_mod.gemv(x, w, t, K, N)) <= oracle_mod.tolerance(w, t, K, N, x))
    gpu.check_error("expert slice")
    Q.cuda_drop(dev)
    L.qg_close(f)


_NAMES = {"EMBED": "token_embd.weight", "LM_HEAD": "output.weight", "FINAL_NORM": "output_norm.weight",
          "Q": "blk.{l}.attn_q.weight", "K": "blk.{l}.attn_k.weight", "V": "blk.{l}.attn_v.weight",
          "O": "blk.{l}.attn_output.weight", "GATE": "blk.{l}.ffn_gate.weight", "UP": "blk.{l}.ffn_up.weight",
          "DOWN": "blk.{l}.ffn_down.weight", "ATTN_NORM": "blk.{l}.attn_norm.weight", "FFN_NORM": "blk.{l}.ffn_norm.weight"}


def _write_model_gguf(path, m, arch="llama"):
    """The tensors of a synthetic HostModel (kept on the host) as a GGUF file with the metadata keys the
    reference reads (src/main.rs:96-215)."""
    import gguf
    from saient_quartz_b200 import synth
    c = m.cfg
    w = gguf.GGUFWriter(path, arch)
    w.add_uint32(f"{arch}.embedding_length", c["embed_dim"])
    w.add_uint32(f"{arch}.attention.head_count", c["n_heads"])
    w.add_uint32(f"{arch}.attention.head_count_kv", c["n_kv_heads"])
    w.add_uint32(f"{arch}.block_count", c["n_layers"])
    w.add_uint32(f"{arch}.feed_forward_length", c["ffn_dim"])
    w.add_float32(f"{arch}.rope.freq_base", c["rope_theta"])
    w.add_uint32(f"{arch}.context_length", c["max_seq"])
    w.add_uint32(f"{arch}.attention.key_length", c["head_dim"])
    w.add_uint32(f"{arch}.vocab_size", c["vocab_size"])
    for (role, layer), (t, arr) in m.host.items():
        name = _NAMES[role].format(l=layer)
        if t == 0:
            w.add_tensor(name, arr.astype(np.float32))
        else:
            in_dim = {"O": c["n_heads"] * c["head_dim"], "DOWN": c["ffn_dim"]}.get(role, c["embed_dim"])
            rb = synth.type_size(t, in_dim)
            w.add_tensor(name, arr.reshape(-1, rb), raw_dtype=gguf.GGMLQuantizationType(t))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


@pytest.mark.gpu
@pytest.mark.parametrize("arch,neox", [("llama", 0), ("qwen2", 1)])
def test_model_from_gguf_equals_model_built_directly(gpu, tmp_path, arch, neox):
    """qh_load_gguf: a model written to a GGUF file and loaded back gives the logits of the model built
    tensor by tensor, bit for bit; the configuration (RoPE convention by architecture included) is derived
    from the metadata."""
    from saient_quartz_b200.host_model import HostModel, Q4K_M_TYPES
    cfg = dict(vocab_size=320, embed_dim=2048, n_heads=16, n_kv_heads=4, n_layers=2, ffn_dim=4096, head_dim=128,
               rope_theta=500000.0, max_seq=64, rope_neox=neox)
    a = HostModel(repack=True, keep_host=True, types=Q4K_M_TYPES, **cfg)
    a.fill_synthetic()
    path = str(tmp_path / "model.gguf")
    _write_model_gguf(path, a, arch)
    b = HostModel.from_gguf(path, max_seq=64)
    for k in ("vocab_size", "embed_dim", "n_heads", "n_kv_heads", "n_layers", "ffn_dim", "head_dim", "max_seq", "rope_neox"):
        assert b.cfg[k] == cfg[k], k
    assert b.cfg["rope_theta"] == 500000.0 and b.cfg["n_experts"] == 0
    for (tok, pos) in ((5, 0), (17, 1), (300, 2)):
        la = a.step(tok, pos, fused=True)
        lb = b.step(tok, pos, fused=True)
        assert np.array_equal(la, lb), (tok, pos)
    assert np.array_equal(a.step(9, 3, fused=False), b.step(9, 3, fused=False))
    gpu.check_error()
    a.close()
    b.close()


@pytest.mark.gpu
def test_model_from_gguf_reports_what_is_missing(gpu, tmp_path):
    import gguf
    from saient_quartz_b200.host_model import HostModel
    path = str(tmp_path / "broken.gguf")
    w = gguf.GGUFWriter(path, "llama")
    w.add_uint32("llama.embedding_length", 256)
    w.add_uint32("llama.attention.head_count", 4)
    w.add_uint32("llama.block_count", 1)
    w.add_uint32("llama.feed_forward_length", 512)
    w.add_uint32("llama.vocab_size", 32)
    w.add_tensor("output_norm.weight", np.ones(256, np.float32))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    with pytest.raises(RuntimeError, match="token_embd.weight"):
        HostModel.from_gguf(path)
