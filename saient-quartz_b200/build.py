"""Build in-tree, from ONE compilation of csrc/quartz_b200.cu for sm_100a:
  saient-quartz_b200/libquartz_b200.so  the CUDA library (what the tests and the benchmark load)
  saient-quartz_b200/libkernels.a       the same object as a static archive under the name the reference's
                                        build.rs links (`static=kernels` + `cudart`, build.rs:52-72)
and saient-quartz_b200/libquartz_host.so (the C++ host side of the decode step, a pure client of the C ABI)."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libquartz_b200.so")
ARCHIVE = os.path.join(HERE, "libkernels.a")
OBJ = os.path.join(HERE, "kernels.o")
HOST_LIB = os.path.join(HERE, "libquartz_host.so")
HOST_SRC = os.path.join(HERE, "host", "forward_state.cpp")


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh")))


def up_to_date():
    if not os.path.exists(LIB) or not os.path.exists(ARCHIVE):
        return False
    t = os.path.getmtime(LIB)
    hdr = os.path.join(HERE, "..", "include", "quartz_b200.h")
    return all(os.path.getmtime(s) <= t for s in sources() + [hdr])


def build_host(force=False):
    hdrs = [os.path.join(HERE, "host", "forward_state.h"), os.path.join(HERE, "host", "gguf_loader.h"),
            os.path.join(HERE, "..", "include", "quartz_b200.h")]
    srcs = [HOST_SRC, os.path.join(HERE, "host", "gguf_loader.cpp"), os.path.join(HERE, "host", "model_loader.cpp")]
    if (not force and os.path.exists(HOST_LIB)
            and all(os.path.getmtime(p) <= os.path.getmtime(HOST_LIB) for p in srcs + [LIB] + hdrs)):
        return HOST_LIB
    tmp = HOST_LIB + ".tmp"
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-o", tmp] + srcs + ["-L" + HERE, "-lquartz_b200",
           "-Wl,-rpath,$ORIGIN"]
    subprocess.check_call(cmd)
    os.replace(tmp, HOST_LIB)   # a reader never sees a half-written library
    return HOST_LIB


def build(force=False, verbose=False):
    if not force and up_to_date():
        build_host()
        return LIB
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    arch = os.environ.get("QUARTZ_CUDA_ARCH", "sm_100a")   # same variable as the reference's build.rs:33
    cc = arch.replace("sm_", "compute_")
    cmd = [nvcc, "-O3", "-std=c++17", "-gencode", f"arch={cc},code={arch}", "-lineinfo", "-Xcompiler", "-fPIC", "-c",
           "-o", OBJ] + [s for s in sources() if s.endswith(".cu")]
    cmd += os.environ.get("QUARTZ_NVCC_FLAGS", "").split()   # extra compiler flags (e.g. -DNAME=value)
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    subprocess.check_call(cmd)
    tmp = LIB + ".tmp"
    subprocess.check_call([nvcc, "-gencode", f"arch={cc},code={arch}", "-shared", "-o", tmp, OBJ])
    os.replace(tmp, LIB)   # a reader never sees a half-written library
    tmp = ARCHIVE + ".tmp"
    if os.path.exists(tmp):
        os.remove(tmp)
    subprocess.check_call(["ar", "rcs", tmp, OBJ])
    os.replace(tmp, ARCHIVE)
    build_host(force=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
