"""One rank of the row-sharded exchange test; launched by test_gpu_mgpu.py (one process per GPU) as
    python -m torch.distributed.run --nproc-per-node G tests/mgpu_worker.py
Every rank uploads its row shard of each matrix, runs cuda_gemv_push + quartz_mgpu_wait, and checks the
COMPLETE vector in its own window against the CPU oracle.  Then a batched block goes through
cuda_gemm + cuda_push_rows, the NCCL all-gather form of the exchange (quartz_nccl_* / quartz_mgpu_allgather), and
last a wait that nobody answers must come back with QZ_ERR_TIMEOUT."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    q = entry.load_package()
    from saient_quartz_b200 import synth
    from saient_quartz_b200.shard import PeerWindow, shard_rows, shard_bytes
    from saient_quartz_b200.iq_tables import load_tables
    import oracle
    oracle.set_tables(load_tables())
    L = q.lib()
    torch.cuda.set_device(local)
    assert L.quartz_set_device(local) == 0
    if world > 1:
        dist.init_process_group("gloo")
    q.ensure_iq_grids()
    win = PeerWindow(L, rank, world, 4 << 20, dist if world > 1 else None)

    def download(off, n):
        out = np.empty(n, dtype=np.float32)
        L.cuda_d2h(out.ctypes.data, win.data_ptr + 4 * off, 4 * n)
        return out

    # (type, K, N, repack): streaming kernels with the fused push epilogue, a raw-layout matrix, and an
    # F16 matrix that takes the any-shape kernel + copy push; two alternating window regions
    cases = [(12, 4096, 14336, True), (14, 14336, 4096, True), (8, 4096, 4096, True), (17, 4096, 1536, True),
             (12, 4096, 1000, False), (1, 512, 301, False)]
    region = [0, 32768]
    for i, (t, K, N, repack) in enumerate(cases):
        w = synth.make_weights(t, K, N, tensor_id=900 + i)
        x = synth.make_x(K, tensor_id=950 + i).reshape(-1)
        n0, n1, per = shard_rows(N, rank, world)
        b0, b1 = shard_bytes(t, K, N, rank, world)
        dw = q.GpuBuf.upload(w[b0:b1]) if n1 > n0 else None
        if repack and dw is not None:
            L.cuda_repack_weights(t, dw.ptr, K, n1 - n0, 1)
        dx = q.GpuBuf.upload(x)
        off = region[i & 1]
        for rep in range(2):   # twice: the counters advance, the result must not change
            if dw is not None:
                win.gemv_push(t, dw.ptr, dx.ptr, off + n0, K, n1 - n0)
            else:
                win.gemv_push(t, 0, dx.ptr, off + n0, K, 0)
            win.wait()
            L.cuda_sync()
            q.check_error("gemv_push")
            y = download(off, N)
            ref = oracle.gemv(x, w, t, K, N)
            tol = 1e-3 * oracle.row_norms(w, t, K, N) * float(np.linalg.norm(x.astype(np.float64)))
            err = np.abs(y.astype(np.float64) - ref)
            assert np.all(err <= tol), f"rank {rank} case {i} rep {rep}: err/tol {np.max(err / np.maximum(tol, 1e-30))}"
            # the exchange is not allowed to run ahead into the region just read: alternate regions
            off = region[(i + rep + 1) & 1]
        if dw is not None:
            dw.drop()
        dx.drop()

    # batched block: Y[M, N] column-sharded, pushed with cuda_push_rows
    t, K, N, M = 12, 2048, 768, 24
    w = synth.make_weights(t, K, N, tensor_id=990)
    X = synth.make_x(K, tensor_id=991, rows=M)
    n0, n1, per = shard_rows(N, rank, world)
    b0, b1 = shard_bytes(t, K, N, rank, world)
    dw, dx = q.GpuBuf.upload(w[b0:b1]), q.GpuBuf.upload(X)
    dy = q.GpuBuf.alloc_f32(M * (n1 - n0))
    L.cuda_gemm(t, dw.ptr, dx.ptr, dy.ptr, M, K, n1 - n0)
    win.push_rows(dy.ptr, M, n1 - n0, 65536 + n0, N)
    win.wait()
    L.cuda_sync()
    q.check_error("gemm push")
    Y = download(65536, M * N).reshape(M, N)
    ref = oracle.gemm(X, w, t, K, N, M)
    norms = oracle.row_norms(w, t, K, N)
    for m in range(M):
        tol = 1e-3 * norms * float(np.linalg.norm(X[m].astype(np.float64)))
        assert np.all(np.abs(Y[m].astype(np.float64) - ref[m]) <= tol), f"rank {rank} gemm token {m}"

    # the same block, and larger ones, with the exchange in the GEMM's own epilogue (cuda_gemm_push): the tensor-core
    # tiles go from the accumulators straight into every rank's window; ragged row counts, several token tiles,
    # Q4_K (raw layout), Q6_K (plane layout, 256-row tiles at 128+ tokens)
    for ci, (t, K, N, M) in enumerate([(12, 2048, 768, 24), (14, 2048, 1000, 300), (12, 4096, 1536, 130)]):
        w = synth.make_weights(t, K, N, tensor_id=992 + ci)
        X = synth.make_x(K, tensor_id=996 + ci, rows=M)
        n0, n1, per = shard_rows(N, rank, world)
        b0, b1 = shard_bytes(t, K, N, rank, world)
        dwp, dxp = q.GpuBuf.upload(w[b0:b1]), q.GpuBuf.upload(X)
        if t == 14:
            L.cuda_repack_weights(t, dwp.ptr, K, n1 - n0, 1)
        off = 500000 if ci & 1 else 65536
        for rep in range(2):
            L.cuda_vec_zero(win.data_ptr + 4 * off, M * N)
            L.cuda_sync()
            if world > 1:
                dist.barrier()   # nobody pushes into a region another rank is still clearing
            assert L.cuda_gemm_push(t, dwp.ptr, dxp.ptr, M, K, n1 - n0, off + n0, N) == 1, L.quartz_error_string()
            win.wait()
            L.cuda_sync()
            q.check_error("gemm push (epilogue)")
            Y = download(off, M * N).reshape(M, N)
            ref = oracle.gemm(X, w, t, K, N, M)
            norms = oracle.row_norms(w, t, K, N)
            for m in range(M):
                tol = 1e-3 * norms * float(np.linalg.norm(X[m].astype(np.float64)))
                assert np.all(np.abs(Y[m].astype(np.float64) - ref[m]) <= tol), f"rank {rank} gemm_push case {ci} token {m}"
            if world > 1:
                dist.barrier()
        dwp.drop()
        dxp.drop()
    # a single token is not taken by the tensor-core kernel: nothing is launched, the caller uses the GEMV form
    assert L.cuda_gemm_push(12, dw.ptr, dx.ptr, 1, 2048, 8, 65536, 768) == 0

    # a chain whose second GEMV reads the first one's gathered output, the wait fused into its conversion
    K, N1, N2 = 2048, 4096, 1024
    wa, wb = synth.make_weights(12, K, N1, tensor_id=970), synth.make_weights(14, N1, N2, tensor_id=971)
    x = synth.make_x(K, tensor_id=972).reshape(-1)
    a0, a1, _ = shard_rows(N1, rank, world)
    c0, c1, _ = shard_rows(N2, rank, world)
    s0, s1 = shard_bytes(12, K, N1, rank, world)
    da = q.GpuBuf.upload(wa[s0:s1])
    s0, s1 = shard_bytes(14, N1, N2, rank, world)
    db = q.GpuBuf.upload(wb[s0:s1])
    L.cuda_repack_weights(14, db.ptr, N1, c1 - c0, 1)
    dx = q.GpuBuf.upload(x)
    RA, RB = 200000, 210000
    for rep in range(3):
        win.gemv_push(12, da.ptr, dx.ptr, RA + a0, K, a1 - a0)
        win.wait(fused=True)
        win.gemv_push(14, db.ptr, win.data_ptr + 4 * RA, RB + c0, N1, c1 - c0)
        win.wait()
        L.cuda_sync()
        q.check_error("chain")
        y1 = download(RA, N1)
        y2 = download(RB, N2)
        ref1 = oracle.gemv(x, wa, 12, K, N1)
        tol1 = 1e-3 * oracle.row_norms(wa, 12, K, N1) * float(np.linalg.norm(x.astype(np.float64)))
        assert np.all(np.abs(y1 - ref1) <= tol1), f"rank {rank} chain y1"
        ref2 = oracle.gemv(y1, wb, 14, N1, N2)
        tol2 = 1e-3 * oracle.row_norms(wb, 14, N1, N2) * float(np.linalg.norm(y1.astype(np.float64)))
        assert np.all(np.abs(y2 - ref2) <= tol2), f"rank {rank} chain y2"
    # several independent sharded GEMVs and their exchange as ONE launch (cuda_gemv_batch_push) + one wait
    import ctypes as C
    bcases = [(12, 4096, 14336), (14, 14336, 4096), (8, 4096, 4096), (12, 4096, 1024)]
    ops, keep, offs, base_off = [], [], [], 300000
    for i, (t, K, N) in enumerate(bcases):
        w = synth.make_weights(t, K, N, tensor_id=930 + i)
        x = synth.make_x(K, tensor_id=940 + i).reshape(-1)
        n0, n1, per = shard_rows(N, rank, world)
        b0, b1 = shard_bytes(t, K, N, rank, world)
        dw = q.GpuBuf.upload(w[b0:b1])
        L.cuda_repack_weights(t, dw.ptr, K, n1 - n0, 1)
        dxb, dummy = q.GpuBuf.upload(x), q.GpuBuf.alloc_f32(max(n1 - n0, 1))
        ops.append(q.chain_op(t, [dw.ptr], [dummy.ptr], K, n1 - n0, 0, 3, dxb.ptr))
        offs.append(base_off + n0)
        keep.append((t, K, N, w, x, dw, dxb, dummy, base_off))
        base_off += (N + 63) & ~63
    arr = (q.ChainOp * len(ops))(*ops)
    off_arr = (C.c_size_t * len(ops))(*offs)
    for rep in range(3):
        if rep == 2:    # the exchange completed inside the kernel itself: no wait launch
            L.quartz_mgpu_wait_in_next_push()
        assert L.cuda_gemv_batch_push(len(ops), arr, off_arr) == 1
        if rep < 2:
            win.wait()
        L.cuda_sync()
        q.check_error("batch push")
        for (t, K, N, w, x, dw, dxb, dummy, o) in keep:
            y = download(o, N)
            ref = oracle.gemv(x, w, t, K, N)
            tol = 1e-3 * oracle.row_norms(w, t, K, N) * float(np.linalg.norm(x.astype(np.float64)))
            assert np.all(np.abs(y.astype(np.float64) - ref) <= tol), f"rank {rank} batch push {t} {K}->{N} rep {rep}"
        if world > 1:
            dist.barrier()   # nobody starts the next round while a slower rank still reads this one

    # a whole row-sharded FFN as ONE launch per rank (cuda_gemv_chain_push): gate/up shards -> exchange inside the
    # kernel -> SwiGLU of the complete vectors -> down shard -> exchange, one wait at the end
    Kf, Ff = 4096, 14336
    OFFG, OFFO = 400000, 440000
    wg, wu = synth.make_weights(12, Kf, Ff, tensor_id=950), synth.make_weights(12, Kf, Ff, tensor_id=951)
    wd = synth.make_weights(14, Ff, Kf, tensor_id=952)
    xf = synth.make_x(Kf, tensor_id=953).reshape(-1)
    f0, f1, _ = shard_rows(Ff, rank, world)
    k0, k1, _ = shard_rows(Kf, rank, world)
    gb0, gb1 = shard_bytes(12, Kf, Ff, rank, world)
    db0, db1 = shard_bytes(14, Ff, Kf, rank, world)
    dwg, dwu, dwd = q.GpuBuf.upload(wg[gb0:gb1]), q.GpuBuf.upload(wu[gb0:gb1]), q.GpuBuf.upload(wd[db0:db1])
    L.cuda_repack_weights(12, dwg.ptr, Kf, f1 - f0, 1)
    L.cuda_repack_weights(12, dwu.ptr, Kf, f1 - f0, 1)
    L.cuda_repack_weights(14, dwd.ptr, Ff, k1 - k0, 1)
    dxf, dumf = q.GpuBuf.upload(xf), q.GpuBuf.alloc_f32(Ff)
    fops = [q.chain_op(12, [dwg.ptr, dwu.ptr], [dumf.ptr, dumf.ptr], Kf, f1 - f0, 0, 3, dxf.ptr),
            q.chain_op(14, [dwd.ptr], [dumf.ptr], Ff, k1 - k0, 0, 2, win.data_ptr + 4 * OFFG, win.data_ptr + 4 * (OFFG + Ff))]
    farr = (q.ChainOp * 2)(*fops)
    foff = (C.c_size_t * 2)(OFFG + f0, OFFO + k0)
    fstr = (C.c_size_t * 2)(Ff, 0)
    for rep in range(2):
        assert L.cuda_gemv_chain_push(2, farr, foff, fstr) == 1, L.quartz_error_string()
        win.wait()
        L.cuda_sync()
        q.check_error("chain push")
        g, u, out = download(OFFG, Ff), download(OFFG + Ff, Ff), download(OFFO, Kf)
        xn = float(np.linalg.norm(xf.astype(np.float64)))
        for got, w in ((g, wg), (u, wu)):
            ref = oracle.gemv(xf, w, 12, Kf, Ff)
            assert np.all(np.abs(got.astype(np.float64) - ref) <= 1e-3 * oracle.row_norms(w, 12, Kf, Ff) * xn), f"rank {rank} chain push gate/up rep {rep}"
        h = (g.astype(np.float64) / (1.0 + np.exp(-g.astype(np.float64))) * u.astype(np.float64)).astype(np.float32)
        ref = oracle.gemv(h, wd, 14, Ff, Kf)
        told = 1e-3 * oracle.row_norms(wd, 14, Ff, Kf) * float(np.linalg.norm(h.astype(np.float64)))
        assert np.all(np.abs(out.astype(np.float64) - ref) <= told), f"rank {rank} chain push down rep {rep}"
        if world > 1:
            dist.barrier()

    # the NCCL form of the exchange through the C ABI: every rank computes its slice into place, ncclAllGather
    idb = C.create_string_buffer(L.quartz_nccl_id_bytes())
    if rank == 0:
        assert L.quartz_nccl_unique_id(idb) == 0, L.quartz_error_string()
    if world > 1:
        box = [idb.raw]
        dist.broadcast_object_list(box, src=0)
        idb = C.create_string_buffer(box[0], len(box[0]))
    assert L.quartz_nccl_init(rank, world, idb) == 0, L.quartz_error_string()
    t, K, N = 12, 4096, 1024 * world
    w = synth.make_weights(t, K, N, tensor_id=980)
    x = synth.make_x(K, tensor_id=981).reshape(-1)
    n0, n1, per = shard_rows(N, rank, world)
    b0, b1 = shard_bytes(t, K, N, rank, world)
    dw, dxx, dyy = q.GpuBuf.upload(w[b0:b1]), q.GpuBuf.upload(x), q.GpuBuf.alloc_f32(per * world)
    for rep in range(2):
        L.cuda_gemv(t, dw.ptr, dxx.ptr, dyy.ptr + 4 * rank * per, K, n1 - n0)
        L.quartz_mgpu_allgather(dyy.ptr + 4 * rank * per, dyy.ptr, per)
        L.cuda_sync()
        q.check_error("nccl all-gather")
        y = dyy.download()[:N]
        ref = oracle.gemv(x, w, t, K, N)
        tol = 1e-3 * oracle.row_norms(w, t, K, N) * float(np.linalg.norm(x.astype(np.float64)))
        assert np.all(np.abs(y.astype(np.float64) - ref) <= tol), f"rank {rank} nccl all-gather"
    L.quartz_nccl_shutdown()

    if world > 1:
        dist.barrier()
        # rank 0 pushes once more and waits, nobody answers: the bounded wait runs out and reports it
        if rank == 0:
            win.gemv_push(12, 0, dx.ptr, 0, 2048, 0)
            win.wait()
            L.cuda_sync()
            assert L.quartz_last_error() == 7, L.quartz_last_error()   # QZ_ERR_TIMEOUT
            L.quartz_clear_error()
        dist.barrier()
    win.close()
    print(f"rank {rank}/{world}: ok", flush=True)


if __name__ == "__main__":
    main()
