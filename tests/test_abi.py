"""CPU tests of the drop-in boundary: the shared library loads without a GPU and
exports every symbol include/quartz_b200.h declares; host-side helpers."""
import ctypes
import os

import numpy as np


def test_library_exports_every_declared_symbol(pkg):
    L = ctypes.CDLL(pkg.library_path())
    declared = pkg.declared_symbols()
    assert len(declared) >= 28
    for name in declared:
        assert hasattr(L, name), f"{name} declared in include/quartz_b200.h but not exported"


def test_reference_call_surface_is_complete(pkg):
    """The 28 functions of the reference's extern "C" block (src/cuda.rs:6-55)."""
    declared = set(pkg.declared_symbols())
    assert len(pkg.REFERENCE_SYMBOLS) == 28
    assert set(pkg.REFERENCE_SYMBOLS) <= declared
    L = pkg.lib()
    for name in pkg.REFERENCE_SYMBOLS:
        assert getattr(L, name) is not None


def test_error_state_starts_clean(pkg):
    L = pkg.lib()
    L.quartz_clear_error()
    assert L.quartz_last_error() == 0
    assert L.quartz_error_string() == b""


def test_missing_library_fails_loudly(pkg, tmp_path, monkeypatch):
    import saient_quartz_b200 as q
    monkeypatch.setattr(q, "_lib", None)
    monkeypatch.setattr(q._build, "LIB", str(tmp_path / "nope.so"))
    try:
        q.lib()
    except RuntimeError as e:
        assert "no CPU fallback" in str(e)
    else:
        raise AssertionError("loading a missing library must raise")


def test_expert_slice_arithmetic(pkg):
    """src/cuda.rs:250-257: expert e starts at e * ggml_type_size(type, K*N)."""
    buf = pkg.GpuBuf(0x1000, 0)
    s = pkg.gpu_expert_slice(buf, 17, 3, 4096 * 14336)
    assert s.ptr == 0x1000 + 3 * 16_973_824 and s.ggml_type == 17
    buf.ptr = None


def test_synthetic_tensors_are_deterministic(pkg):
    from saient_quartz_b200 import synth
    a = synth.make_weights(12, 512, 8)
    b = synth.make_weights(12, 512, 8)
    assert np.array_equal(a, b) and a.size == synth.type_size(12, 512 * 8)
    d = a.reshape(-1, 144)[:, 0:2].copy().view(np.float16).astype(np.float32)
    assert d.min() >= 9.9e-5 and d.max() <= 1.001e-3
    sc = synth.make_weights(14, 512, 8).reshape(-1, 210)[:, 192:208].view(np.int8)
    assert sc.min() >= -32 and sc.max() <= 31
    assert synth.algorithmic_bytes(12, 4096, 4096) == 9_469_952
    assert synth.algorithmic_bytes(14, 4096, 128256) == 431_469_568
