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


def test_static_archive_links_like_the_reference_build(pkg, tmp_path):
    """build.rs:52-72 of the reference links `static=kernels` and `cudart`: a C program that takes the address of
    every declared symbol must link against libkernels.a the same way."""
    import shutil
    import subprocess
    from saient_quartz_b200 import build as b
    assert os.path.exists(b.ARCHIVE), "libkernels.a was not built"
    names = pkg.declared_symbols()
    src = tmp_path / "link_test.c"
    src.write_text("".join(f"extern void {n}(void);\n" for n in names) +
                   "int main(void) { void (*p[])(void) = {" + ", ".join(names) + "}; return p[0] == 0; }\n")
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    exe = tmp_path / "link_test"
    cc = shutil.which("gcc")
    assert cc
    subprocess.check_call([cc, str(src), "-o", str(exe), "-L" + os.path.dirname(b.ARCHIVE), "-lkernels",
                           "-L" + os.path.join(cuda, "lib64"), "-lcudart", "-lstdc++", "-lm", "-lpthread", "-ldl"])
    assert exe.exists()


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
