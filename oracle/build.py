"""Build recipe for the CPU oracle (test infrastructure, never shipped).

  oracle/libquartz_oracle.so   C restatement of the reference's src/dequant.rs
  oracle/_ref/libkernels_ref.so  the reference's OWN src/cuda_kernels.cu, compiled
                               unmodified for sm_100a from where it lies in the
                               mounted reference tree (only when that tree is
                               present; nothing is copied into this repository).

The reference's CPU path is Rust and there is no Rust toolchain here, so the
CPU side of oracle/_ref cannot be built; its CUDA side is one self-contained
.cu file and can.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "libquartz_oracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libkernels_ref.so")


def reference_root():
    """Where the reference project is mounted: the environment variable QUARTZ_REFERENCE_ROOT, else a
    directory named `reference` beside this repository; None when neither exists."""
    cand = os.environ.get("QUARTZ_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return cand if os.path.isdir(os.path.join(cand, "src")) else None



def _newer(target, *sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources if os.path.exists(s))


def build_oracle(force=False):
    src = os.path.join(HERE, "dequant_ref.c")
    hdr = os.path.join(HERE, "dequant_ref.h")
    if not force and _newer(ORACLE_SO, src, hdr):
        return ORACLE_SO
    # -ffp-contract=off: the Rust reference never fuses a*b+c; -mavx2 -mfma mirrors
    # its #[target_feature(enable = "avx2,fma")] build and changes no result.
    cmd = ["gcc", "-O3", "-std=c11", "-fPIC", "-shared", "-ffp-contract=off", "-mavx2", "-mfma",
           "-fopenmp", "-o", ORACLE_SO, src, "-lm"]
    subprocess.check_call(cmd)
    return ORACLE_SO


def build_ref(force=False):
    """Compile the reference's CUDA kernels (GPU A/B baseline and secondary check)."""
    root = reference_root()
    ref_cu = os.path.join(root, "src", "cuda_kernels.cu") if root else None
    if not ref_cu or not os.path.exists(ref_cu):
        return REF_SO if os.path.exists(REF_SO) else None
    if not force and _newer(REF_SO, ref_cu):
        return REF_SO
    os.makedirs(REF_DIR, exist_ok=True)
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    cmd = [nvcc, "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC",
           "-o", REF_SO, ref_cu]
    subprocess.check_call(cmd, stderr=subprocess.DEVNULL)
    return REF_SO


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    print(build_ref(force="--force" in sys.argv))
