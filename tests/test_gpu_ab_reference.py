"""A/B timing on the same GPU: this library's cuda_gemv against the reference's own CUDA kernels
(oracle/_ref/libkernels_ref.so, compiled unmodified from the reference's src/cuda_kernels.cu for
sm_100a), shape by shape, same weights, back-to-back launches rotating over enough distinct
weight copies to exceed the L2.  Prints a markdown table (run with -s) and writes it to ab_reference.md
in the report directory ($QUARTZ_REPORT_DIR); asserts only that no streaming format is slower than the
reference."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

SHAPES = [(12, 4096, 4096), (12, 4096, 1024), (12, 4096, 14336), (14, 14336, 4096), (14, 4096, 128256), (8, 4096, 4096),
          (6, 4096, 14336), (7, 4096, 14336), (2, 4096, 14336), (3, 4096, 14336), (13, 4096, 14336), (10, 4096, 14336),
          (20, 4096, 14336), (16, 4096, 14336), (17, 4096, 14336), (22, 4096, 14336), (18, 4096, 14336),
          (21, 4096, 14336), (12, 8192, 28672), (14, 28672, 8192)]


def test_ab_against_reference_kernels(gpu, oracle_mod, tables):
    import torch
    from saient_quartz_b200 import synth
    R = oracle_mod.ref_kernels()
    if R is None:
        pytest.skip("oracle/_ref not built (reference tree was not mounted at build time)")
    for name in ("iq3s", "iq2s", "iq2xxs", "iq2xs"):
        getattr(R, f"cuda_set_{name}_grid")(tables[name].ctypes.data)
    R.cuda_set_ksigns(tables["ksigns"].ctypes.data)
    L = gpu.lib()

    def loop(fn, reps):
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(reps):
            fn(i)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) * 1e3 / reps

    lines = ["| format | shape | this library µs | GB/s | reference kernels µs | GB/s | ratio |", "|---|---|---|---|---|---|---|"]
    for t, K, N in SHAPES:
        nbytes = synth.type_size(t, K * N)
        copies = max(2, min(12, int(400e6 / nbytes) + 1))
        raw, rep = [], []
        for c in range(copies):
            w = synth.make_weights(t, K, N, tensor_id=900 + c)
            raw.append(gpu.GpuBuf.upload(w))
            b = gpu.GpuBuf.upload(w)
            L.cuda_repack_weights(t, b.ptr, K, N, 1)
            rep.append(b)
        dx, dy = gpu.GpuBuf.upload(synth.make_x(K)), gpu.GpuBuf.alloc_f32(N)
        mine = loop(lambda i: L.cuda_gemv(t, rep[i % copies].ptr, dx.ptr, dy.ptr, K, N), 2 * copies)
        by = synth.algorithmic_bytes(t, K, N)
        if t in (2, 3, 18):     # formats the reference does not have
            lines.append(f"| {synth.FORMATS[t][0]} | {K}->{N} | {mine:.1f} | {by / mine / 1e3:.0f} | - | - | - |")
            continue
        ref = loop(lambda i: R.cuda_gemv(t, raw[i % copies].ptr, dx.ptr, dy.ptr, K, N), 2 * copies)
        R.cuda_sync()
        lines.append(f"| {synth.FORMATS[t][0]} | {K}->{N} | {mine:.1f} | {by / mine / 1e3:.0f} | {ref:.1f} | "
                     f"{by / ref / 1e3:.0f} | {ref / mine:.1f}x |")
        assert mine <= ref * 1.05, (t, K, N, mine, ref)
    gpu.check_error()
    table = "\n".join(lines)
    print("\n" + table)
    out_dir = os.environ.get("QUARTZ_REPORT_DIR")   # where to leave the table as a file, if anywhere
    if out_dir:
        os.makedirs(out_dir, exist_ok=True)
        with open(os.path.join(out_dir, "ab_reference.md"), "w") as f:
            f.write(table + "\n")
