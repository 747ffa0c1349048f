#!/usr/bin/env python
"""Benchmark of the quantized-weight dequant-GEMV hot path on B200.

Workload (N=1): the mixed-format GEMV sweep at Llama-3-8B decode shapes, batch 1 --
Q4_K 4096->4096, Q4_K 4096->1024, Q4_K 4096->14336, Q6_K 14336->4096,
Q6_K 4096->128256, Q8_0 4096->4096 -- on seeded synthetic GGUF-layout weights
(543 MB of distinct weight bytes per step, > the 126 MB L2, so every step streams from
HBM) and f32 activations ~ N(0,1).  One step = one pass over the six GEMVs.

  value      algorithmic GB/s of the whole step, operands resident in HBM: the faster of six
             cuda_gemv calls (graph replay) and cuda_gemv_batch (one conversion kernel + one
             persistent kernel); both are reported (six_separate_calls, batched_single_launch)
  e2e        host to host: page-locked arenas, cuda_h2d_async, the six GEMVs, cuda_d2h_async,
             replayed as one graph, cuda_sync per step; beside it the reference's own call
             sequence (GpuScratch.gemv: cuda_h2d, cuda_gemv, cuda_d2h, cuda_sync per GEMV,
             src/cuda.rs:107-127)
  roofline   the dominant kernel (Q6_K streaming GEMV at the lm_head shape) against the
             measured HBM copy bandwidth in MEASURED_PEAKS.json
  cpu_baseline  the CPU oracle (C port of the reference's src/dequant.rs gemv, rows over
             all host cores) on the same six shapes
  gemv_shapes, decode (generation loop, prefill), gemm, moe_ffn, sharded70b, sharded_gemm:
             the other configurations of the baseline, each checked against the oracle

N>1 (torchrun, one rank per GPU): every matrix is row-sharded over the output dimension;
each rank computes its slices and stores them into every rank's window from the kernel's
epilogue (peer stores over NVLink): cuda_gemv_batch_push runs a rank's six shard GEMVs, their
exchange and its wait as one persistent launch (the headline), six cuda_gemv_push calls and
the NCCL all-gather form are timed beside it; total work is fixed ("strong" scaling).

--impl reference times the CPU oracle alone (the reference has no buildable CPU
binary here: its host is Rust and there is no Rust toolchain).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "dequant-GEMV HBM GB/s"
UNIT = "GB/s"
WORKLOAD = "llama3-8b-decode-gemv-sweep(Q4_K 4096x4096,4096x1024,4096x14336; Q6_K 14336x4096,4096x128256; Q8_0 4096x4096), batch 1"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--small", action="store_true", help="profiling case: lm_head cut to 40080 rows (134 MB, still larger than L2; ~0.3 GB on the device)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true", help="skip the Llama-3-8B-shaped decode-step section")
    ap.add_argument("--no-moe", action="store_true", help="skip the batched MoE FFN section")
    ap.add_argument("--no-sharded", action="store_true", help="skip the 70B-shaped row-sharded pair section")
    ap.add_argument("--no-gemm", action="store_true", help="skip the batched (prefill) dequant-GEMM section")
    ap.add_argument("--decode-only", action="store_true",
                    help="profiling case: run only the fused decode-step section (no CPU parity pass) and print it")
    ap.add_argument("--moe-only", action="store_true", help="profiling case: run only the batched MoE FFN section and print its rows")
    ap.add_argument("--gemm-only", default=None, metavar="FORMAT:M",
                    help="profiling case: run only this dequant-GEMM case (e.g. Q4_K:2048) and print its row")
    return ap.parse_args()


def sweep(small=False):
    from saient_quartz_b200 import synth
    shapes = list(synth.LLAMA3_8B_GEMV_SWEEP)
    if small:
        shapes = [(l, t, k, (40080 if n == 128256 else n)) for (l, t, k, n) in shapes]
    return shapes


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows = []
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                for nm, v in zip(names, r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(nm)
            except Exception:
                continue
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_pass(oracle, mats, xs, threads=0):
    t0 = time.perf_counter()
    for (label, t, K, N), w, x in zip(mats["shapes"], mats["w"], xs):
        oracle.gemv(x, w, t, K, N, threads)
    return time.perf_counter() - t0


def make_host_tensors(shapes, rank=0, world=1):
    """Seeded weights (this rank's row shard) and activations for every shape."""
    from saient_quartz_b200 import synth
    ws, xs = [], []
    for i, (label, t, K, N) in enumerate(shapes):
        w = synth.make_weights(t, K, N, tensor_id=100 + i)
        if world > 1:
            rb = synth.type_size(t, K)
            n0, n1 = shard_rows(N, rank, world)
            w = w[n0 * rb:n1 * rb]
        ws.append(w)
        xs.append(synth.make_x(K, tensor_id=200 + i))
    return {"shapes": shapes, "w": ws}, xs


def shard_rows(N, rank, world):
    from saient_quartz_b200.shard import shard_rows as _sr
    return _sr(N, rank, world)[:2]


def run_reference(args):
    """The reference's CPU implementation of the path (C port of src/dequant.rs gemv), all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # all the host threads this process may use (a multi-process launcher may have exported OMP_NUM_THREADS=1)
    os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))
    import __graft_entry__ as entry
    entry.load_package()
    import oracle
    from saient_quartz_b200 import synth
    shapes = sweep(args.small)
    mats, xs = make_host_tensors(shapes)
    total_bytes = sum(synth.algorithmic_bytes(t, K, N) for (_, t, K, N) in shapes)
    for _ in range(max(args.warmup, 1)):
        cpu_pass(oracle, mats, xs)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_pass(oracle, mats, xs)
    dt = (time.perf_counter() - t0) / args.steps
    val = total_bytes / dt / 1e9
    cores = oracle.max_threads()
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD + (" [small]" if args.small else ""), "hardware": "host CPU"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": "the full six-shape sweep, every step (C port of src/dequant.rs gemv, one task per output row)"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def gemv_shape_rows(q, L, torch, np, shapes, mats, xs, with_ref, want_parity):
    """One row per shape of the sweep: cuda_gemv (activation conversion included) over rotating copies of the
    matrix that together exceed the L2, recorded as one graph and replayed, so the figure is graph-amortised
    and HBM-fed.  With with_ref the reference's own CUDA kernels (built unmodified for sm_100a, when they were
    built) run the same shape in the same loop, eagerly, as the same-box GPU baseline; with want_parity every
    shape's output is checked against the CPU oracle."""
    from saient_quartz_b200 import synth
    peak, _ = peaks()
    R = None
    if with_ref:
        import oracle
        from saient_quartz_b200.iq_tables import load_tables
        R = oracle.ref_kernels()
        if R is not None:
            tb = load_tables()
            for name in ("iq3s", "iq2s", "iq2xxs", "iq2xs"):
                getattr(R, f"cuda_set_{name}_grid")(tb[name].ctypes.data)
            R.cuda_set_ksigns(tb["ksigns"].ctypes.data)
    rows = []
    for (label, t, K, N), w, x in zip(shapes, mats["w"], xs):
        nbytes = synth.type_size(t, K * N)
        copies = max(2, min(96, int(np.ceil(260e6 / nbytes))))
        bufs = []
        for _ in range(copies):
            b = q.GpuBuf.upload(w)
            L.cuda_repack_weights(t, b.ptr, K, N, 1)
            bufs.append(b)
        dx, dy = q.GpuBuf.upload(x), q.GpuBuf.alloc_f32(N)

        def run():
            for b in bufs:
                L.cuda_gemv(t, b.ptr, dx.ptr, dy.ptr, K, N)
        run()
        L.cuda_sync()
        g = None
        if L.quartz_graph_begin():
            run()
            g = L.quartz_graph_end()
        q.check_error("per-shape graph capture")
        fn = (lambda: L.quartz_graph_launch(g)) if g else run
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        reps = 5
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (reps * copies)
        by = synth.algorithmic_bytes(t, K, N)
        row = {"shape": label, "us": us, "gbs": by / us / 1e3, "frac_of_measured_hbm": by / us / 1e3 / peak,
               "frac_of_8TBs_nominal": by / us / 1e3 / 8000.0, "copies": copies,
               "launch": "graph replay" if g else "eager"}
        if g:
            L.quartz_graph_destroy(g)
        if want_parity:
            import oracle
            ref = oracle.gemv(x, w, t, K, N)
            tol = oracle.tolerance(w, t, K, N, x)
            err = np.abs(dy.download().astype(np.float64) - ref)
            row["max_err_over_tolerance"] = float(np.max(err / tol))
            assert np.all(err <= tol), f"bench output of {label} failed the parity bound"
        if R is not None:
            raw = [q.GpuBuf.upload(w) for _ in range(min(copies, 24))]
            for i in range(3):
                R.cuda_gemv(t, raw[i % len(raw)].ptr, dx.ptr, dy.ptr, K, N)
            torch.cuda.synchronize()
            n = 2 * len(raw)
            e0.record()
            for i in range(n):
                R.cuda_gemv(t, raw[i % len(raw)].ptr, dx.ptr, dy.ptr, K, N)
            e1.record()
            torch.cuda.synchronize()
            rus = e0.elapsed_time(e1) * 1e3 / n
            row["ref_cuda_kernels"] = {"us": rus, "gbs": by / rus / 1e3, "launch": "eager",
                                       "what": "the reference's own kernel for this format, compiled unmodified for sm_100a"}
            for b in raw:
                b.drop()
        for b in bufs + [dx, dy]:
            b.drop()
        q.check_error("per-shape rows")
        rows.append(row)
    return rows


def gemm_section(q, args, torch, np, want_parity, only=None):
    """Batched dequant-GEMM for prefill: Q4_K 4096->14336 and Q6_K 14336->4096 times M = 16, 64, 512, 2048
    f32 activations ~ N(0,1) (bf16 inside the tensor-core tile, f32 accumulation in TMEM); the bf16-activation
    entry point is timed beside it."""
    from saient_quartz_b200 import synth
    L = q.lib()
    peaks_file = os.path.join(ROOT, "MEASURED_PEAKS.json")
    tf_burst, tf_sust = 1590.0, 1400.0
    if os.path.exists(peaks_file):
        try:
            pk = json.load(open(peaks_file))
            tf_burst, tf_sust = float(pk["bf16_tflops"]), float(pk["bf16_tflops_sustained"])
        except Exception:
            pass
    hbm, _ = peaks()
    out = []
    for (t, K, N) in ((12, 4096, 14336), (14, 14336, 4096)):
        if only and synth.FORMATS[t][0] != only[0]:
            continue
        w = synth.make_weights(t, K, N, tensor_id=400 + t)
        dw = q.GpuBuf.upload(w)
        L.cuda_repack_weights(t, dw.ptr, K, N, 1)
        # The small-M rows are HBM-bound by definition, so they must stream from HBM: the timed loop rotates over
        # copies of the matrix that together exceed the 126 MB L2 (one 33 / 48 MB matrix would simply stay in L2).
        n_copies = int(np.ceil(150e6 / w.nbytes)) + 1
        extra = []
        for _ in range(n_copies - 1):
            b = q.GpuBuf.upload(w)
            L.cuda_repack_weights(t, b.ptr, K, N, 1)
            extra.append(b)
        ring = [dw] + extra
        for M in (16, 64, 512, 2048):
            if only and M != only[1]:
                continue
            X = synth.make_x(K, tensor_id=410, rows=M)
            dx, dy = q.GpuBuf.upload(X), q.GpuBuf.alloc_f32(M * N)
            for _ in range(2):
                L.cuda_gemm(t, dw.ptr, dx.ptr, dy.ptr, M, K, N)
            torch.cuda.synchronize()
            reps = 2 * len(ring) if M <= 64 else 5
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(reps):
                L.cuda_gemm(t, (ring[i % len(ring)] if M <= 64 else dw).ptr, dx.ptr, dy.ptr, M, K, N)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / reps
            q.check_error("gemm")
            flops = 2.0 * M * K * N
            nbytes = synth.type_size(t, K * N) + 4.0 * M * K + 4.0 * M * N
            row = {"format": synth.FORMATS[t][0], "M": M, "K": K, "N": N, "ms": ms, "tflops": flops / ms / 1e9,
                   "gbs": nbytes / ms / 1e6, "frac_of_measured_bf16_burst": flops / ms / 1e9 / tf_burst,
                   "frac_of_measured_bf16_sustained": flops / ms / 1e9 / tf_sust,
                   "frac_of_measured_hbm": nbytes / ms / 1e6 / hbm, "bound": "hbm" if M <= 64 else "tensor"}
            # the same GEMM fed bf16 activations (cuda_gemm_bf16: what a host that keeps bf16 activations calls)
            xb16 = torch.from_numpy(X).to(torch.bfloat16).cuda().contiguous()
            for _ in range(2):
                L.cuda_gemm_bf16(t, dw.ptr, xb16.data_ptr(), dy.ptr, M, K, N)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(reps):
                L.cuda_gemm_bf16(t, dw.ptr, xb16.data_ptr(), dy.ptr, M, K, N)
            e1.record()
            torch.cuda.synchronize()
            row["ms_bf16_activations"] = e0.elapsed_time(e1) / reps
            q.check_error("gemm bf16")
            L.cuda_gemm(t, dw.ptr, dx.ptr, dy.ptr, M, K, N)   # (the parity check below reads the f32 form's output)
            if want_parity and M in (16, 512):
                import oracle
                y = dy.download().reshape(M, N)
                pick = [0, M - 1]
                ref = oracle.gemm(X[pick], w, t, K, N, 2)
                norms = oracle.row_norms(w, t, K, N)
                worst = 0.0
                for i, mrow in enumerate(pick):
                    tol = 1e-3 * norms * float(np.linalg.norm(X[mrow].astype(np.float64)))
                    worst = max(worst, float(np.max(np.abs(y[mrow].astype(np.float64) - ref[i]) / tol)))
                row["max_err_over_tolerance"] = worst
                assert worst <= 1.0, f"GEMM parity failed: {row}"
                if M == 16:   # the CPU path's gemm() on the same 16 tokens, all host threads
                    tc0 = time.perf_counter()
                    oracle.gemm(X, w, t, K, N, M)
                    row["cpu_oracle_ms"] = (time.perf_counter() - tc0) * 1e3
                    row["cpu_cores"] = oracle.max_threads()
            if M <= 64:
                row["weights"] = f"rotating over {len(ring)} copies of the matrix (> L2): every launch streams from HBM"
            out.append(row)
            dx.drop(); dy.drop()
        for b in ring:
            b.drop()
    return out


def decode_section(q, args, torch, np, want_parity, fused_only=False):
    """Full batch-1 decode of a random-init Llama-3-8B-architecture model in the fixed Q4_K_M-style layout
    (q/k/v/o/gate/up Q4_K, down + output head Q6_K), f32 KV cache pre-filled with N(0,1) at context 1024.
    The headline leg is a GENERATION LOOP: 64 consecutive positions 1024..1087 with 64 different token ids;
    the step is recorded once (token id and position are device words) and replayed per token."""
    from saient_quartz_b200.host_model import HostModel, LLAMA3_8B
    L = q.lib()
    t0 = time.perf_counter()
    m = HostModel(keep_host=want_parity, **LLAMA3_8B)
    m.fill_synthetic()
    kv = m.fill_kv(1024, keep=want_parity)
    build_s = time.perf_counter() - t0
    pos0, n_gen = 1024, 64
    rng = np.random.Generator(np.random.PCG64([0x5EED0001, 4242]))
    tokens = [int(v) for v in rng.integers(0, LLAMA3_8B["vocab_size"], size=n_gen)]
    kv_bytes = 32 * 2 * 1025 * 1024 * 4
    bytes_per_token = m.weight_bytes + kv_bytes
    out = {"model": "llama-3-8b architecture, random init, Q4_K_M-style layout", "context": 1024,
           "bytes_per_token": bytes_per_token, "build_s": round(build_s, 1)}
    peak, _ = peaks()

    def rates(ms):
        return {"tok_s": 1e3 / ms, "ms_per_token": ms, "gbs": bytes_per_token / (ms * 1e-3) / 1e9,
                "frac_of_measured_hbm": bytes_per_token / (ms * 1e-3) / 1e9 / peak}

    for name, fused in (("chained_graph", 2), ("fused_graph", 1), ("reference_sequence", 0)):
        if fused_only and not fused:
            continue
        # device time of a generation loop: every step another token and the next position
        n = n_gen if fused else 8
        for i in range(3):
            m.step_device(tokens[i], pos0 + i, fused)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n):
            m.step_device(tokens[i], pos0 + i, fused)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / n
        out[name] = dict(rates(ms), launches_per_token=m.launches(), steps_timed=n,
                         what="generation loop: consecutive positions from 1024, a different token id per step")
        if fused:
            # the same step replayed with a FIXED (token, position): what a replay-only figure would read
            e0.record()
            for i in range(20):
                m.step_device(tokens[0], pos0, fused)
            e1.record()
            torch.cuda.synchronize()
            out[name]["fixed_position_replay_ms"] = e0.elapsed_time(e1) / 20
            out[name]["graphs_recorded"] = m.graphs_recorded()
        q.check_error("decode " + name)
    if fused_only:
        m.close()
        return out
    best = 2 if out["chained_graph"]["ms_per_token"] <= out["fused_graph"]["ms_per_token"] else 1
    # THE decode figure: generation loop, host to host -- token id in, 513 KB of logits out, every step,
    # including whatever graph work the host does
    logits = None
    m.step(tokens[0], pos0, fused=best)
    t1 = time.perf_counter()
    for i in range(n_gen):
        logits = m.step(tokens[i], pos0 + i, fused=best)
    wall = time.perf_counter() - t1
    out["generation_loop"] = dict(rates(wall / n_gen * 1e3), sequence="chained" if best == 2 else "fused", steps=n_gen,
                                  positions=[pos0, pos0 + n_gen - 1], graphs_recorded=m.graphs_recorded(),
                                  what="host to host: per step the token id goes in and 513 KB of logits come out; host wall clock")
    out["e2e_tok_s"] = out["generation_loop"]["tok_s"]
    out["e2e_sequence"] = out["generation_loop"]["sequence"]
    if want_parity:
        import oracle
        from oracle.forward_ref import RefModel
        from saient_quartz_b200.iq_tables import load_tables
        oracle.set_tables(load_tables())
        # (1) the first step of the loop against the CPU oracle, from the seeded cache alone
        r = RefModel(m.cfg, m.host)
        for l, (k, v) in enumerate(kv):
            r.set_kv(l, k, v)
        first = m.step(tokens[0], pos0, fused=best)
        t2 = time.perf_counter()
        want = r.forward(tokens[0], pos0)
        cpu_s = time.perf_counter() - t2
        rel = float(np.abs(first.astype(np.float64) - want).max() / np.abs(want).max())
        out["parity_max_rel_err_vs_cpu_oracle"] = rel
        out["cpu_oracle_tok_s"] = 1.0 / cpu_s
        assert rel < 5e-3, f"decode-step logits differ from the CPU oracle: {rel}"
        # (2) the LAST step of the loop: the oracle takes the cache rows the 63 steps before it appended on
        # the device (a CPU replay of all 64 steps would take a minute) and must reproduce its logits
        m.fill_kv(1024)
        for i in range(n_gen):
            logits = m.step(tokens[i], pos0 + i, fused=best)
        r2 = RefModel(m.cfg, m.host)
        for l, (k, v) in enumerate(kv):
            k2, v2 = m.read_kv(l, pos0, n_gen - 1)
            r2.set_kv(l, np.concatenate([k, k2]), np.concatenate([v, v2]))
        want = r2.forward(tokens[-1], pos0 + n_gen - 1)
        rel = float(np.abs(logits.astype(np.float64) - want).max() / np.abs(want).max())
        out["generation_loop"]["last_step_max_rel_err_vs_cpu_oracle"] = rel
        assert rel < 5e-3, f"last step of the generation loop differs from the CPU oracle: {rel}"
    # batched prefill of a 512-token prompt (tensor-core GEMMs over the whole prompt, batched RoPE / KV append, causal
    # prompt attention): host wall clock from the token ids to the last token's logits; against it, the same 512
    # tokens through the replayed decode step would take 512 x ms_per_token
    n_prompt = 512
    prompt = [int(v) for v in rng.integers(0, LLAMA3_8B["vocab_size"], size=n_prompt)]
    try:
        m.prefill(prompt, pos0=0)
        t3 = time.perf_counter()
        for _ in range(3):
            m.prefill(prompt, pos0=0)
        pw = (time.perf_counter() - t3) / 3
        q.check_error("prefill")
        out["prefill"] = {"tokens": n_prompt, "ms": pw * 1e3, "tok_s": n_prompt / pw,
                          "vs_token_by_token_decode": (n_prompt * out["fused_graph"]["ms_per_token"] * 1e-3) / pw,
                          "what": "qh_prefill: 512-token prompt from position 0, host to host (token ids in, last token's logits out)"}
    except RuntimeError as e:   # (a model the batched path does not take would fall here; this one is taken)
        out["prefill"] = {"error": str(e)}
    m.close()
    return out


def moe_section(q, args, torch, np):
    """Mixtral-style MoE FFN, batched: 8 experts, top-2 routing from a softmax over N(0,1) router logits,
    256 tokens, expert matrices 4096->14336 (gate, up) and 14336->4096 (down) in IQ3_XXS and in IQ2_XS."""
    from saient_quartz_b200 import synth
    L = q.lib()
    q.ensure_iq_grids()
    K, F, E, top_k, M = 4096, 14336, 8, 2, 256
    rng = np.random.Generator(np.random.PCG64([0x5EED0001, 77]))
    logits = rng.standard_normal((M, E)).astype(np.float32)
    ids = np.ascontiguousarray(np.argsort(-logits, axis=1)[:, :top_k].astype(np.int32))
    sel = np.take_along_axis(logits, ids, axis=1)
    w = np.exp(sel - sel.max(axis=1, keepdims=True))
    w = np.ascontiguousarray((w / w.sum(axis=1, keepdims=True)).astype(np.float32))
    X = synth.make_x(K, tensor_id=500, rows=M)
    dx, dout = q.GpuBuf.upload(X), q.GpuBuf.alloc_f32(M * K)
    hbm, _ = peaks()
    out = []
    for t in (18, 17):
        bufs = []
        for which, (kk, nn) in enumerate(((K, F), (K, F), (F, K))):
            blob = np.concatenate([synth.make_weights(t, kk, nn, tensor_id=510 + 10 * which + e) for e in range(E)])
            b = q.GpuBuf.upload(blob)
            L.cuda_repack_weights(t, b.ptr, kk, nn, E)
            bufs.append(b)
            del blob

        def call():
            L.cuda_moe_ffn(t, t, bufs[0].ptr, bufs[1].ptr, bufs[2].ptr, dx.ptr, dout.ptr, M, K, F, E, top_k,
                           ids.ctypes.data, w.ctypes.data, 0)
        for _ in range(2):
            call()
        torch.cuda.synchronize()
        reps = 5
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            call()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        q.check_error("moe")
        wbytes = 3 * E * synth.type_size(t, K * F)
        flops = 2.0 * M * top_k * K * F * 3
        out.append({"format": synth.FORMATS[t][0], "tokens": M, "experts": E, "top_k": top_k, "ms": ms,
                    "weight_bytes": wbytes, "gbs": (wbytes + 8.0 * M * K) / ms / 1e6, "tflops": flops / ms / 1e9,
                    "frac_of_measured_hbm": (wbytes + 8.0 * M * K) / ms / 1e6 / hbm,
                    "tokens_per_expert": [int((ids == e).sum()) for e in range(E)]})
        for b in bufs:
            b.drop()
    dx.drop(); dout.drop()
    return out


def sharded70b_section(q, L, torch, win, rank, world, dist, steps, cpu_baseline=False):
    """Llama-3-70B-shaped FFN pair, row-sharded over the ranks: Q4_K 8192->28672 whose complete output
    (gathered in every rank's window by the GEMV's own peer stores) is the activation of Q6_K
    28672->8192.  Batch 1 through cuda_gemv_push, batch 32 through cuda_gemm + cuda_push_rows; the
    NCCL all-gather form of batch 1 is timed beside it.  Times are max over ranks, on the device."""
    from saient_quartz_b200 import synth
    from saient_quartz_b200.shard import shard_rows as sr, shard_bytes
    K1, N1, N2 = 8192, 28672, 8192
    out = {"shapes": "Q4_K 8192->28672 -> Q6_K 28672->8192", "n_gpus": world}
    w1, w2 = synth.make_weights(12, K1, N1, tensor_id=300), synth.make_weights(14, N1, N2, tensor_id=301)
    a0, a1, per1 = sr(N1, rank, world)
    b0, b1, per2 = sr(N2, rank, world)
    s0, s1 = shard_bytes(12, K1, N1, rank, world)
    d1 = q.GpuBuf.upload(w1[s0:s1])
    s0, s1 = shard_bytes(14, N1, N2, rank, world)
    d2 = q.GpuBuf.upload(w2[s0:s1])
    if world == 1 and cpu_baseline:
        # the CPU path's gemv on the same pair, all host threads (second call of each: warm)
        import oracle
        x1 = synth.make_x(K1, tensor_id=302).reshape(-1)
        oracle.gemv(x1, w1, 12, K1, N1)
        tc = time.perf_counter()
        h = oracle.gemv(x1, w1, 12, K1, N1)
        oracle.gemv(h, w2, 14, N1, N2)
        tc = time.perf_counter() - tc
        out["batch1_cpu_oracle"] = {"ms": tc * 1e3, "gbs": (synth.algorithmic_bytes(12, K1, N1) +
                                                             synth.algorithmic_bytes(14, N1, N2)) / tc / 1e9,
                                    "cores": oracle.max_threads()}
    del w1
    L.cuda_repack_weights(12, d1.ptr, K1, a1 - a0, 1)
    L.cuda_repack_weights(14, d2.ptr, N1, b1 - b0, 1)
    total = synth.algorithmic_bytes(12, K1, N1) + synth.algorithmic_bytes(14, N1, N2)
    M = 32
    X = synth.make_x(K1, tensor_id=302, rows=M)
    dx = q.GpuBuf.upload(X)
    A, B = 0, M * N1                       # window regions (floats): Y1 [M x N1], Y2 [M x N2]
    base = win.data_ptr

    def timed(fn, n):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / n
        if world > 1:
            tt = torch.tensor([ms], device="cuda")
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms = float(tt.item())
        q.check_error("sharded 70B-shaped pair")
        return ms

    def chain1():
        # the wait for an exchange runs inside the activation conversion of the GEMV that consumes it (the first
        # GEMV of an iteration thereby also completes the previous iteration's second exchange)
        win.wait(fused=True)
        win.gemv_push(12, d1.ptr, dx.ptr, A + a0, K1, a1 - a0)
        win.wait(fused=True)
        win.gemv_push(14, d2.ptr, base + 4 * A, B + b0, N1, b1 - b0)

    fn = chain1
    g = None
    if L.quartz_graph_begin():
        chain1()
        g = L.quartz_graph_end()
        q.check_error("sharded graph capture")
        if g:
            fn = lambda: L.quartz_graph_launch(g)   # noqa: E731
    n = max(10, min(steps, 50))
    ms = timed(fn, n)
    win.wait()
    out["batch1_push"] = {"ms": ms, "gbs": total / (ms * 1e-3) / 1e9, "launch": "graph replay" if g else "eager",
                          "exchange": "peer stores from the GEMV epilogue; flag wait fused into the consumer's activation conversion"}
    if g:
        L.quartz_graph_destroy(g)

    # the same pair as ONE launch per rank: both GEMVs and the exchange between them inside the persistent kernel
    # (cuda_gemv_chain_push), one wait for the last exchange
    import ctypes as C
    import numpy as np
    dummy = q.GpuBuf.alloc_f32(max(a1 - a0, b1 - b0, 1))
    pops = [q.chain_op(12, [d1.ptr], [dummy.ptr], K1, a1 - a0, 0, 3, dx.ptr),
            q.chain_op(14, [d2.ptr], [dummy.ptr], N1, b1 - b0, 0, 3, base + 4 * A)]
    parr = (q.ChainOp * 2)(*pops)
    poff = (C.c_size_t * 2)(A + a0, B + b0)

    def pair_one_launch():
        ok = L.cuda_gemv_chain_push(2, parr, poff, None)
        win.wait()
        return ok
    sup = torch.tensor([1 if pair_one_launch() else 0], device="cuda")
    if world > 1:
        dist.all_reduce(sup, op=dist.ReduceOp.MIN)
    torch.cuda.synchronize()
    q.check_error("sharded pair, one launch")
    if int(sup.item()) == 1:
        fn, g = pair_one_launch, None
        if L.quartz_graph_begin():
            pair_one_launch()
            g = L.quartz_graph_end()
            q.check_error("sharded pair graph capture")
            if g:
                fn = lambda: L.quartz_graph_launch(g)   # noqa: E731
        ms = timed(fn, n)
        out["batch1_one_launch"] = {"ms": ms, "gbs": total / (ms * 1e-3) / 1e9, "launch": "graph replay" if g else "eager",
                                    "launches_per_step": 2,
                                    "exchange": "cuda_gemv_chain_push: both GEMVs in one persistent kernel per rank; the first "
                                                "exchange is published and polled inside the kernel, the second completed by one wait"}
        if g:
            L.quartz_graph_destroy(g)
        if rank == 0:
            # what was just timed, against the CPU oracle: the second GEMV of the complete first output
            import oracle
            from saient_quartz_b200.iq_tables import load_tables
            oracle.set_tables(load_tables())
            h = np.empty(N1, dtype=np.float32)
            y = np.empty(N2, dtype=np.float32)
            L.cuda_d2h(h.ctypes.data, base + 4 * A, 4 * N1)
            L.cuda_d2h(y.ctypes.data, base + 4 * B, 4 * N2)
            ref = oracle.gemv(h, w2, 14, N1, N2)
            assert np.all(np.abs(y - ref) <= oracle.tolerance(w2, 14, N1, N2, h)), "sharded one-launch pair failed the parity bound"
            out["batch1_one_launch"]["parity"] = "second GEMV of the gathered first output within the oracle bound"
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()   # the other ranks must not start the next exchange while rank 0 is still in the oracle
    del w2
    dummy.drop()

    if world > 1:
        y1 = torch.zeros(per1 * world, dtype=torch.float32, device="cuda")
        y2 = torch.zeros(per2 * world, dtype=torch.float32, device="cuda")

        def chain_nccl():
            L.cuda_gemv(12, d1.ptr, dx.ptr, y1.data_ptr() + 4 * rank * per1, K1, a1 - a0)
            dist.all_gather_into_tensor(y1, y1[rank * per1:(rank + 1) * per1])
            L.cuda_gemv(14, d2.ptr, y1.data_ptr(), y2.data_ptr() + 4 * rank * per2, N1, b1 - b0)
            dist.all_gather_into_tensor(y2, y2[rank * per2:(rank + 1) * per2])
        ms = timed(chain_nccl, n)
        out["batch1_nccl_allgather"] = {"ms": ms, "gbs": total / (ms * 1e-3) / 1e9, "launch": "eager"}

    dy1 = q.GpuBuf.alloc_f32(M * (a1 - a0))
    dy2 = q.GpuBuf.alloc_f32(M * (b1 - b0))

    def chain32():
        L.cuda_gemm(12, d1.ptr, dx.ptr, dy1.ptr, M, K1, a1 - a0)
        win.push_rows(dy1.ptr, M, a1 - a0, A + a0, N1)
        win.wait()
        L.cuda_gemm(14, d2.ptr, base + 4 * A, dy2.ptr, M, N1, b1 - b0)
        win.push_rows(dy2.ptr, M, b1 - b0, B + b0, N2)
        win.wait()
    ms = timed(chain32, max(5, n // 2))
    flops = 2.0 * M * (K1 * N1 + N1 * N2)
    out["batch32_push"] = {"ms": ms, "gbs": total / (ms * 1e-3) / 1e9, "tflops": flops / ms / 1e9, "launch": "eager"}
    for b in (d1, d2, dx, dy1, dy2):
        b.drop()
    return out


def sharded_gemm_section(q, L, torch, win, rank, world, dist):
    """The prefill GEMMs row-sharded over the ranks: Q4_K 4096->14336 and Q6_K 14336->4096 times M = 16, 64, 512,
    2048 tokens.  Every rank holds the rows [n0, n1) of the matrix and computes its [M, n1-n0] block; the block goes
    into every rank's window from the GEMM's own epilogue (cuda_gemm_push) or, timed beside it, by a copy kernel after
    the GEMM (cuda_gemm + cuda_push_rows); after the wait each rank holds the complete [M, N] output.
    Times are device times, max over ranks; TFLOP/s and GB/s are whole-job figures."""
    from saient_quartz_b200 import synth
    from saient_quartz_b200.shard import shard_rows as sr, shard_bytes
    out = []
    for (t, K, N) in ((12, 4096, 14336), (14, 14336, 4096)):
        w = synth.make_weights(t, K, N, tensor_id=400 + t)
        n0, n1, per = sr(N, rank, world)
        b0, b1 = shard_bytes(t, K, N, rank, world)
        dw = q.GpuBuf.upload(w[b0:b1])
        del w
        L.cuda_repack_weights(t, dw.ptr, K, n1 - n0, 1)
        for M in (16, 64, 512, 2048):
            X = synth.make_x(K, tensor_id=410, rows=M)
            dx, dy = q.GpuBuf.upload(X), q.GpuBuf.alloc_f32(M * (n1 - n0))

            def step_copy():
                L.cuda_gemm(t, dw.ptr, dx.ptr, dy.ptr, M, K, n1 - n0)
                win.push_rows(dy.ptr, M, n1 - n0, n0, N)
                win.wait()

            def step():   # the exchange in the GEMM's epilogue
                if not L.cuda_gemm_push(t, dw.ptr, dx.ptr, M, K, n1 - n0, n0, N):
                    L.cuda_gemm(t, dw.ptr, dx.ptr, dy.ptr, M, K, n1 - n0)
                    win.push_rows(dy.ptr, M, n1 - n0, n0, N)
                win.wait()
            reps = 10 if M <= 64 else 5

            def timed_ms(fn):
                for _ in range(3):
                    fn()
                torch.cuda.synchronize()
                if world > 1:
                    dist.barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(reps):
                    fn()
                e1.record()
                torch.cuda.synchronize()
                v = e0.elapsed_time(e1) / reps
                if world > 1:
                    tt = torch.tensor([v], device="cuda")
                    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                    v = float(tt.item())
                return v
            ms_copy = timed_ms(step_copy)
            ms = timed_ms(step)
            q.check_error("sharded gemm")
            flops = 2.0 * M * K * N
            nbytes = synth.type_size(t, K * N) + 4.0 * M * K + 4.0 * M * N
            # what must cross NVLink INTO every rank: the other ranks' blocks of the f32 output
            link_bytes = 4.0 * M * N * (world - 1) / world
            row = {"format": synth.FORMATS[t][0], "M": M, "K": K, "N": N, "n_gpus": world, "ms": ms,
                   "tflops": flops / ms / 1e9, "gbs": nbytes / ms / 1e6,
                   "exchange": "cuda_gemm_push: peer stores from the GEMM's epilogue + one wait",
                   "ms_gemm_then_copy_kernel": ms_copy}
            if world > 1:
                # roofline of the fused kernel: the slower of flops / measured bf16 peak and link bytes / 770 GB/s
                t_link, t_flop = link_bytes / 770e9 * 1e3, flops / world / 1.6156e15 * 1e3
                row["nvlink_bytes_in_per_rank"] = link_bytes
                row["frac_of_fused_roofline"] = max(t_link, t_flop) / ms
            out.append(row)
            dx.drop(); dy.drop()
        dw.drop()
    return out


def main():
    args = parse_args()
    if args.impl == "reference":
        return run_reference(args)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    # one GPU per process; every GPU of the box stays visible so that peers' windows can be mapped
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    ids = vis.split(",") if vis else None
    dev = local_rank if world > 1 else 0
    phys_index = ids[dev] if ids and dev < len(ids) else str(dev)

    import numpy as np
    import torch
    import __graft_entry__ as entry
    q = entry.load_package()
    from saient_quartz_b200 import synth
    L = q.lib()
    torch.cuda.set_device(dev)
    if L.quartz_set_device(dev) != 0:
        q.check_error("quartz_set_device")
    if args.decode_only:
        print(json.dumps({"decode": decode_section(q, args, torch, np, False, fused_only=True)}))
        return
    if args.moe_only:
        print(json.dumps({"moe_ffn": moe_section(q, args, torch, np)}))
        return
    if args.gemm_only:
        name, m = args.gemm_only.split(":")
        print(json.dumps({"gemm": gemm_section(q, args, torch, np, False, only=(name, int(m)))}))
        return
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{dev}"))
    else:
        dist = None
    from saient_quartz_b200.shard import PeerWindow

    shapes = sweep(args.small)
    mats, xs = make_host_tensors(shapes, rank, world)
    total_bytes = sum(synth.algorithmic_bytes(t, K, N) for (_, t, K, N) in shapes)

    # device residency: weights (repacked once, as the loader would), x, y
    d_w, d_x, y_full, rows, y_off = [], [], [], [], []
    off = 0
    for (label, t, K, N), w, x in zip(shapes, mats["w"], xs):
        n0, n1 = shard_rows(N, rank, world)
        buf = q.GpuBuf.upload(w)
        L.cuda_repack_weights(t, buf.ptr, K, n1 - n0, 1)
        d_w.append(buf)
        d_x.append(q.GpuBuf.upload(x))
        per = (N + world - 1) // world
        y_full.append(torch.zeros(per * world, dtype=torch.float32, device="cuda"))
        rows.append((n0, n1, per))
        y_off.append(off)            # this shape's region of the exchange window, in floats
        off += (N + 63) & ~63
    # exchange window: the six output vectors (sweep) or the 70B-shaped pair at batch 32, whichever is larger
    half = off
    win_floats = max(2 * half, 32 * (28672 + 8192))
    if world > 1 and not args.small and not args.no_sharded:
        win_floats = max(win_floats, 2048 * 14336)   # the complete output of the largest sharded prefill GEMM
    win, win_err = None, None
    if world > 1 or not args.small:
        try:
            win = PeerWindow(L, rank, world, 4 * win_floats, dist)
        except RuntimeError as e:      # no inter-process peer mapping on this box: NCCL carries the exchange
            win_err = str(e)
            L.quartz_clear_error()
        if world > 1:
            ok = torch.tensor([1 if win is not None else 0], device="cuda")
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok.item()) == 0 and win is not None:
                win.close()
                win = None
    L.cuda_sync()
    q.check_error("setup")

    def step_nccl():
        for i, (label, t, K, N) in enumerate(shapes):
            n0, n1, per = rows[i]
            L.cuda_gemv(t, d_w[i].ptr, d_x[i].ptr, y_full[i].data_ptr() + 4 * rank * per, K, n1 - n0)
            if world > 1:
                dist.all_gather_into_tensor(y_full[i], y_full[i][rank * per:(rank + 1) * per])

    step_no = [0]

    def step_push(parity=None):
        # every rank's slice lands in every rank's window from the GEMV's own epilogue; the six GEMVs of a
        # step do not depend on one another, so one wait at the end of the step covers the six exchanges.
        # Two sets of regions alternate from step to step: a rank one step ahead never writes what a slower
        # rank may still be reading.
        par = step_no[0] & 1 if parity is None else parity
        step_no[0] += 1
        for i, (label, t, K, N) in enumerate(shapes):
            n0, n1, per = rows[i]
            win.gemv_push(t, d_w[i].ptr, d_x[i].ptr, par * half + y_off[i] + n0, K, n1 - n0)
        win.wait()

    step = step_push if (world > 1 and win is not None) else step_nccl

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    sync_all()
    q.check_error("warmup")
    graph = None
    if world == 1 or win is not None:   # (NCCL calls run on another stream and are not part of a recording)
        # what a host would do with a fixed call sequence: record the six GEMV calls (and, sharded, their
        # exchanges) once (quartz_graph_begin/end) and replay them; kernels become programmatic dependents
        graph2 = None
        if L.quartz_graph_begin():
            step(0) if (world > 1 and win is not None) else step()
            graph = L.quartz_graph_end()
        if graph and world > 1 and win is not None and L.quartz_graph_begin():
            step(1)
            graph2 = L.quartz_graph_end()
        q.check_error("graph capture")
        if graph and (world == 1 or win is None or graph2):
            eager_step = step
            replay_no = [0]

            def step():   # noqa: F811
                L.quartz_graph_launch(graph2 if (graph2 and replay_no[0] & 1) else graph)
                replay_no[0] += 1
            for _ in range(4):
                step()
            sync_all()
        else:
            graph = None

    sampler = ClockSampler(phys_index)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    sync_all()
    ms = ev0.elapsed_time(ev1) / args.steps
    if world > 1:
        tt = torch.tensor([ms], device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = float(tt.item())
    q.check_error("timed region")

    # ---- dominant kernel: the streaming GEMV at the largest shape, timed on the launching stream ----
    # Back-to-back launches over two distinct copies of the matrix (each far larger than the 126 MB
    # L2, so every launch streams from HBM); the activation is converted once, outside the loop, so
    # the events bracket launches of gemv_tma_kernel only.  (An explicit L2 flush by a large write
    # is NOT used: the dirty lines it leaves are written back during the next kernel and steal
    # ~25 % of its DRAM bandwidth.)
    import ctypes as C
    dom = max(range(len(shapes)), key=lambda i: synth.type_size(shapes[i][1], shapes[i][2] * shapes[i][3]))
    _, dt_, dK, dN = shapes[dom]
    n0, n1, per = rows[dom]
    dom_bytes = synth.algorithmic_bytes(dt_, dK, n1 - n0)
    second = q.GpuBuf.upload(mats["w"][dom])
    L.cuda_repack_weights(dt_, second.ptr, dK, n1 - n0, 1)
    copies = [(C.c_void_p * 1)(d_w[dom].ptr), (C.c_void_p * 1)(second.ptr)]
    Y1 = (C.c_void_p * 1)(y_full[dom].data_ptr() + 4 * rank * per)
    S1 = (C.c_int * 1)(0)
    L.cuda_quantize_x(d_x[dom].ptr, dK, 0)
    reps = max(10, min(args.steps, 50))
    for i in range(4):
        L.cuda_gemv_q(dt_, 1, copies[i & 1], S1, Y1, dK, n1 - n0, 0)
    torch.cuda.synchronize()
    dom_runs = []
    for _ in range(3):
        a_, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a_.record()
        for i in range(reps):
            L.cuda_gemv_q(dt_, 1, copies[i & 1], S1, Y1, dK, n1 - n0, 0)
        b_.record()
        torch.cuda.synchronize()
        dom_runs.append(a_.elapsed_time(b_) / reps)
    dom_ms = sorted(dom_runs)
    dom_avg = sum(dom_ms) / len(dom_ms)
    peak, peak_src = peaks()
    achieved = dom_bytes / (dom_avg * 1e-3) / 1e9
    second.drop()
    q.check_error("roofline loop")

    # ---- end to end through the reference-facing host path (host x in, host y out) ----
    e2e = None
    if world == 1:
        max_in = max(K for (_, _, K, _) in shapes)
        max_out = max(N for (_, _, _, N) in shapes)
        sc = q.GpuScratch(max_in, max_out)
        pinned = [torch.from_numpy(x).pin_memory() for x in xs]
        hx = [p.numpy() for p in pinned]

        def e2e_step():
            outs = []
            for i, (label, t, K, N) in enumerate(shapes):
                outs.append(sc.gemv(hx[i], d_w[i], t, K, N))
            return outs
        for _ in range(3):
            outs_ref = e2e_step()
        outs_ref = [np.array(o, copy=True) for o in outs_ref]
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_e2e = max(5, args.steps // 2)
        e0.record()
        for _ in range(n_e2e):
            e2e_step()
        e1.record()
        torch.cuda.synchronize()
        seq_ms = e0.elapsed_time(e1) / n_e2e
        q.check_error("e2e (reference call sequence)")
        # the same step as a host would drive it for throughput: inputs in page-locked buffers, the six
        # (copy in, GEMV, copy out) triples recorded once and replayed, one synchronisation per step
        # one page-locked arena for the step's six activation vectors and one for its six outputs, mirrored by
        # one device arena each: two copies per step
        x_off = np.cumsum([0] + [K for (_, _, K, _) in shapes])
        y_off = np.cumsum([0] + [(N + 63) & ~63 for (_, _, _, N) in shapes])
        hx_all = torch.empty(int(x_off[-1]), dtype=torch.float32).pin_memory()
        hy_all = torch.empty(int(y_off[-1]), dtype=torch.float32).pin_memory()
        for i, x in enumerate(xs):
            hx_all[int(x_off[i]):int(x_off[i + 1])] = torch.from_numpy(x.reshape(-1))
        dx_all, dy_all = q.GpuBuf.alloc_f32(int(x_off[-1])), q.GpuBuf.alloc_f32(int(y_off[-1]))
        hy = [hy_all[int(y_off[i]):int(y_off[i]) + N] for i, (_, _, _, N) in enumerate(shapes)]

        def e2e_calls():
            L.cuda_h2d_async(dx_all.ptr, hx_all.data_ptr(), 4 * int(x_off[-1]))
            for i, (label, t, K, N) in enumerate(shapes):
                L.cuda_gemv(t, d_w[i].ptr, dx_all.ptr + 4 * int(x_off[i]), dy_all.ptr + 4 * int(y_off[i]), K, N)
            L.cuda_d2h_async(hy_all.data_ptr(), dy_all.ptr, 4 * int(y_off[-1]))
        e2e_calls()
        L.cuda_sync()
        g2 = None
        if L.quartz_graph_begin():
            e2e_calls()
            g2 = L.quartz_graph_end()
        q.check_error("e2e graph capture")

        def e2e_fast():
            if g2:
                L.quartz_graph_launch(g2)
            else:
                e2e_calls()
            L.cuda_sync()          # the host owns the results again
        for _ in range(3):
            e2e_fast()
        # wall clock: the step ends on the host (after the synchronisation), not on the device
        t_w = time.perf_counter()
        n_fast = max(10, args.steps)
        for _ in range(n_fast):
            e2e_fast()
        e2e_ms = (time.perf_counter() - t_w) / n_fast * 1e3
        q.check_error("e2e")
        i = 1
        assert np.array_equal(hy[i].numpy(), outs_ref[i]), "e2e paths disagree"
        e2e = {"value": total_bytes / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
               "h2d_bytes_per_step": 4 * int(x_off[-1]), "d2h_bytes_per_step": 4 * int(y_off[-1]), "ms_per_step": e2e_ms,
               "how": "page-locked host arenas; cuda_h2d_async (six vectors), cuda_gemv x6, cuda_d2h_async (six outputs) " +
                      ("replayed as one graph" if g2 else "eager") + ", cuda_sync per step; host wall clock",
               "reference_call_sequence": {"value": total_bytes / (seq_ms * 1e-3) / 1e9, "ms_per_step": seq_ms,
                                           "how": "GpuScratch::gemv as in src/cuda.rs:107-127: cuda_h2d, cuda_gemv, cuda_d2h, cuda_sync per GEMV"}}
        if g2:
            L.quartz_graph_destroy(g2)
    # the six GEMVs as ONE launch (they are independent: cuda_gemv_batch streams all six matrices through one
    # persistent kernel without a kernel boundary); reported beside the headline, which stays six cuda_gemv calls
    batched = None
    if world == 1:
        ops = [q.chain_op(t, [d_w[i].ptr], [y_full[i].data_ptr()], K, N, 0, 3, d_x[i].ptr)
               for i, (label, t, K, N) in enumerate(shapes)]
        arr = (q.ChainOp * len(ops))(*ops)
        if L.cuda_gemv_chain_supported(len(ops), arr):
            before = [y.clone() for y in y_full]
            for _ in range(3):
                L.cuda_gemv_batch(len(ops), arr)
            torch.cuda.synchronize()
            same = all(torch.equal(a_, b_) for a_, b_ in zip(before, y_full))
            gb = None
            if L.quartz_graph_begin():
                L.cuda_gemv_batch(len(ops), arr)
                gb = L.quartz_graph_end()
            fnb = (lambda: L.quartz_graph_launch(gb)) if gb else (lambda: L.cuda_gemv_batch(len(ops), arr))
            for _ in range(3):
                fnb()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                fnb()
            e1.record()
            torch.cuda.synchronize()
            bms = e0.elapsed_time(e1) / args.steps
            q.check_error("batched sweep")
            batched = {"ms_per_step": bms, "value": total_bytes / (bms * 1e-3) / 1e9, "unit": UNIT, "launches_per_step": 2,
                       "outputs_identical_to_separate_calls": bool(same),
                       "how": "cuda_gemv_batch: one kernel converts the six activation vectors, one persistent kernel runs the six independent GEMVs; graph replay"}
            if gb:
                L.quartz_graph_destroy(gb)
    elif win is not None:
        # sharded: the six GEMVs of this rank's shards AND their exchange as one launch (cuda_gemv_batch_push), one
        # wait per step; the two window-region parities alternate as in the headline step
        import ctypes as C
        dummy = torch.zeros(max(n1 - n0 for (n0, n1, _) in rows) + 64, dtype=torch.float32, device="cuda")
        ops = [q.chain_op(t, [d_w[i].ptr], [dummy.data_ptr()], K, rows[i][1] - rows[i][0], 0, 3, d_x[i].ptr)
               for i, (label, t, K, N) in enumerate(shapes)]
        arr = (q.ChainOp * len(ops))(*ops)
        offs = [(C.c_size_t * len(ops))(*[par * half + y_off[i] + rows[i][0] for i in range(len(shapes))]) for par in (0, 1)]

        def bstep(par):
            L.quartz_mgpu_wait_in_next_push()   # the persistent kernel completes its own exchange: no wait launch
            return L.cuda_gemv_batch_push(len(ops), arr, offs[par])
        supported = torch.tensor([1 if bstep(0) else 0], device="cuda")
        dist.all_reduce(supported, op=dist.ReduceOp.MIN)
        sync_all()
        if int(supported.item()) == 1:
            bstep(1)
            sync_all()
            gbs = [None, None]
            for par in (0, 1):
                if L.quartz_graph_begin():
                    bstep(par)
                    gbs[par] = L.quartz_graph_end()
            q.check_error("batched sharded graph capture")
            bno = [0]

            def fnb():
                par = bno[0] & 1
                bno[0] += 1
                if gbs[0] and gbs[1]:
                    L.quartz_graph_launch(gbs[par])
                else:
                    bstep(par)
            for _ in range(4):
                fnb()
            sync_all()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                fnb()
            e1.record()
            sync_all()
            tt = torch.tensor([e0.elapsed_time(e1) / args.steps], device="cuda")
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            bms = float(tt.item())
            q.check_error("batched sharded sweep")
            batched = {"ms_per_step": bms, "value": total_bytes / (bms * 1e-3) / 1e9, "unit": UNIT, "launches_per_step": 2,
                       "how": "cuda_gemv_batch_push: one kernel converts the six activation vectors, one persistent kernel runs "
                              "this rank's six shard GEMVs, their peer-store exchange and the wait for the other ranks' slices; "
                              "graph replay; device time, max over ranks"}
            # the complete vectors in this rank's window against the CPU oracle (what was just timed)
            if rank == 0:
                import oracle
                from saient_quartz_b200.iq_tables import load_tables
                oracle.set_tables(load_tables())
                par = (bno[0] - 1) & 1
                for i in (1, 5):
                    _, t, K, N = shapes[i]
                    wfull = synth.make_weights(t, K, N, tensor_id=100 + i)
                    got = np.empty(N, dtype=np.float32)
                    L.cuda_d2h(got.ctypes.data, win.data_ptr + 4 * (par * half + y_off[i]), 4 * N)
                    ref = oracle.gemv(xs[i].reshape(-1), wfull, t, K, N)
                    tol = oracle.tolerance(wfull, t, K, N, xs[i].reshape(-1))
                    assert np.all(np.abs(got - ref) <= tol), "batched sharded bench output failed the parity bound"
            sync_all()   # the other ranks must not start the next exchange while rank 0 is still in the oracle
            for g_ in gbs:
                if g_:
                    L.quartz_graph_destroy(g_)

    nccl_variant = None
    if world > 1 and win is not None:
        # end to end, sharded: every rank copies the step's six activation vectors in (one page-locked arena, one
        # copy), pushes its six slices, waits once and reads the six complete outputs back from its window (one
        # copy); recorded once per region parity and replayed, one synchronisation per step
        kx = np.cumsum([0] + [K for (_, _, K, _) in shapes])
        hx_all = torch.empty(int(kx[-1]), dtype=torch.float32).pin_memory()
        for i, x in enumerate(xs):
            hx_all[int(kx[i]):int(kx[i + 1])] = torch.from_numpy(x.reshape(-1))
        hy_all = torch.empty(half, dtype=torch.float32).pin_memory()
        dx_all = q.GpuBuf.alloc_f32(int(kx[-1]))
        hy = [hy_all[y_off[i]:y_off[i] + N].numpy() for i, (_, _, _, N) in enumerate(shapes)]

        # the six shard GEMVs as one persistent launch where the library takes them that way (every rank agreed above)
        e2e_batch = batched is not None
        if e2e_batch:
            e_ops = [q.chain_op(t, [d_w[i].ptr], [dummy.data_ptr()], K, rows[i][1] - rows[i][0], 0, 3, dx_all.ptr + 4 * int(kx[i]))
                     for i, (label, t, K, N) in enumerate(shapes)]
            e_arr = (q.ChainOp * len(e_ops))(*e_ops)

        def e2e_calls(par):
            L.cuda_h2d_async(dx_all.ptr, hx_all.data_ptr(), 4 * int(kx[-1]))
            if e2e_batch:
                L.quartz_mgpu_wait_in_next_push()
                L.cuda_gemv_batch_push(len(e_ops), e_arr, offs[par])
            else:
                for i, (label, t, K, N) in enumerate(shapes):
                    n0, n1, per = rows[i]
                    win.gemv_push(t, d_w[i].ptr, dx_all.ptr + 4 * int(kx[i]), par * half + y_off[i] + n0, K, n1 - n0)
                win.wait()
            L.cuda_d2h_async(hy_all.data_ptr(), win.data_ptr + 4 * par * half, 4 * half)
        e2e_calls(0)
        e2e_calls(1)
        L.cuda_sync()
        eg = [None, None]
        for par in (0, 1):
            if L.quartz_graph_begin():
                e2e_calls(par)
                eg[par] = L.quartz_graph_end()
        q.check_error("e2e sharded graph capture")
        e2e_no = [0]

        def e2e_step():
            par = e2e_no[0] & 1
            e2e_no[0] += 1
            if eg[0] and eg[1]:
                L.quartz_graph_launch(eg[par])
            else:
                e2e_calls(par)
            L.cuda_sync()
        for _ in range(4):
            e2e_step()
        sync_all()
        n_e2e = max(10, args.steps)
        t_w = time.perf_counter()
        for _ in range(n_e2e):
            e2e_step()
        e2e_ms = (time.perf_counter() - t_w) / n_e2e * 1e3
        tt = torch.tensor([e2e_ms], device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_ms = float(tt.item())
        e2e = {"value": total_bytes / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
               "h2d_bytes_per_step": 4 * int(kx[-1]), "d2h_bytes_per_step": 4 * half, "ms_per_step": e2e_ms,
               "how": "per rank: page-locked arenas, cuda_h2d_async, " + ("cuda_gemv_batch_push (six shards, their exchange and its wait in one persistent launch)" if e2e_batch else "cuda_gemv_push x6, one wait") + ", cuda_d2h_async of the window, "
                      + ("replayed as a graph" if eg[0] and eg[1] else "eager") + ", cuda_sync per step; host wall clock, max over ranks",
               "note": "every rank holds the complete outputs"}
        q.check_error("e2e sharded")
        # parity of what was timed: the complete vector in this rank's window against the CPU oracle
        if rank == 0:
            import oracle
            from saient_quartz_b200.iq_tables import load_tables
            oracle.set_tables(load_tables())
            i = 1
            _, t, K, N = shapes[i]
            wfull = synth.make_weights(t, K, N, tensor_id=100 + i)
            ref = oracle.gemv(xs[i].reshape(-1), wfull, t, K, N)
            tol = oracle.tolerance(wfull, t, K, N, xs[i].reshape(-1))
            assert np.all(np.abs(hy[i] - ref) <= tol), "sharded bench output failed the parity bound"
        # the same step with NCCL's all-gather as the exchange (eager launches)
        for _ in range(3):
            step_nccl()
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step_nccl()
        e1.record()
        sync_all()
        tt = torch.tensor([e0.elapsed_time(e1) / args.steps], device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        nccl_ms = float(tt.item())
        nccl_variant = {"ms_per_step": nccl_ms, "value": total_bytes / (nccl_ms * 1e-3) / 1e9, "unit": UNIT,
                        "exchange": "ncclAllGather of the f32 slices after every GEMV, eager launches"}
        q.check_error("nccl variant")

    clocks = sampler.stop() if rank == 0 else None

    moe = None
    if rank == 0 and world == 1 and not args.small and not args.no_moe:
        moe = moe_section(q, args, torch, np)

    sharded = None
    if win is not None and not args.small and not args.no_sharded:
        sharded = sharded70b_section(q, L, torch, win, rank, world, dist, args.steps, cpu_baseline=not args.no_cpu_baseline)

    sharded_gemm = None
    if win is not None and world > 1 and not args.small and not args.no_sharded:
        sharded_gemm = sharded_gemm_section(q, L, torch, win, rank, world, dist)

    # ---- parity spot check of what was just timed (rank 0, smallest shape) + CPU baseline ----
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        import oracle
        t_budget, passes = 10.0, []
        cpu_pass(oracle, mats, xs)
        t_start = time.perf_counter()
        while time.perf_counter() - t_start < t_budget and len(passes) < 40:
            passes.append(cpu_pass(oracle, mats, xs))
        passes.sort()
        med = passes[len(passes) // 2]
        cpu = {"value": total_bytes / med / 1e9, "unit": UNIT, "cores": oracle.max_threads(), "kind": "port",
               "sample": f"the full six-shape sweep, median of {len(passes)} passes (C port of src/dequant.rs gemv)",
               "ms_per_step": med * 1e3}
        i = 1
        _, t, K, N = shapes[i]
        ref = oracle.gemv(xs[i], mats["w"][i], t, K, N)
        got = y_full[i][:N].cpu().numpy()
        tol = oracle.tolerance(mats["w"][i], t, K, N, xs[i])
        assert np.all(np.abs(got - ref) <= tol), "bench output failed the parity bound"

    shape_rows = None
    if rank == 0 and world == 1:
        shape_rows = gemv_shape_rows(q, L, torch, np, shapes, mats, xs, with_ref=not args.no_cpu_baseline and not args.small,
                                     want_parity=not args.no_cpu_baseline)

    decode = None
    if rank == 0 and world == 1 and not args.small and not args.no_decode:
        decode = decode_section(q, args, torch, np, want_parity=not args.no_cpu_baseline)

    gemm = None
    if rank == 0 and world == 1 and not args.small and not args.no_gemm:
        gemm = gemm_section(q, args, torch, np, want_parity=not args.no_cpu_baseline)

    if rank == 0:
        launches_per_step = len(shapes)   # one streaming GEMV per shape (the activation conversion runs in its prologue)
        if world > 1:
            launches_per_step += 1   # the step's exchange wait
        six_calls = {"ms_per_step": ms, "value": total_bytes / (ms * 1e-3) / 1e9, "unit": UNIT,
                     "how": ("CUDA graph replay of the six cuda_gemv calls" if graph else "six cuda_gemv calls, eager") +
                            ("" if world == 1 else " (cuda_gemv_push per shape, one wait per step)")}
        headline_how = six_calls["how"]
        # The six GEMVs of the sweep do not depend on one another: the public call for that is cuda_gemv_batch
        # (one persistent launch).  The headline is whichever of the two public paths is faster; both are reported.
        if batched and batched["ms_per_step"] < ms:
            ms = batched["ms_per_step"]
            launches_per_step = batched["launches_per_step"]
            headline_how = batched["how"]
        line = {
            "metric": METRIC, "value": total_bytes / (ms * 1e-3) / 1e9, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "i8 dp4a + f32", "data": "synthetic",
            "config": {"workload": WORKLOAD + (" [small]" if args.small else ""),
                       "launch": headline_how,
                       "parallelism": "single GPU" if world == 1 else (
                           f"row-sharded x{world}; output slices exchanged by peer stores from the GEMV epilogue (NVLink), one flag wait per step"
                           if win is not None else f"row-sharded x{world}; NCCL all-gather of the f32 slices after every GEMV (peer windows unavailable: {win_err})"),
                       "l2": "inputs larger than L2: each step streams 543 MB of distinct weights (> 126 MB L2); the roofline loop alternates two 431 MB copies of the matrix",
                       "pct_of_8TBs_nominal": 100.0 * total_bytes / (ms * 1e-3) / 8e12},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": dom_bytes * 1.0006 if world == 1 else None,
                         "traffic_note": "ncu dram__bytes_read.sum of the 134 MB launch (4096->40080) of this kernel = 134.75 MB = 1.0006 x its weight bytes "
                                         "(its write counter also shows 4 MB of write-backs of earlier buffers; the kernel stores 160 KB); "
                                         "scaled by rows to the full launch; captured with gemv_tma.cuh as of commit fe36a7e "
                                         "(profiles/gemv_tma_q6k_q4k_ncu.md)",
                         "kernel": f"gemv_tma_kernel<{synth.FORMATS[dt_][0]}> {dK}->{n1 - n0}",
                         "bytes_per_launch": dom_bytes, "avg_us": dom_avg * 1e3, "min_us": dom_ms[0] * 1e3,
                         "launches_timed": 3 * reps, "frac_of_8TBs_nominal": achieved / 8000.0,
                         "peak_source": peak_src},
            "cpu_baseline": cpu,
            "e2e": e2e if e2e else {"value": total_bytes / (ms * 1e-3) / 1e9, "unit": UNIT, "h2d_bytes_per_step": 0,
                                    "d2h_bytes_per_step": 0, "note": "multi-GPU: operands resident"},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
            "gemv_shapes": shape_rows,
            "decode": decode,
            "gemm": gemm,
            "six_separate_calls": six_calls,
            "batched_single_launch": batched,
            "moe_ffn": moe,
            "sharded70b": sharded,
            "sharded_gemm": sharded_gemm,
            "nccl_allgather_variant": nccl_variant,
        }
        print(json.dumps(line))
    if win is not None:
        win.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
