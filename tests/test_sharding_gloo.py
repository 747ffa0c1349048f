"""CPU test of the multi-GPU path's host logic: two gloo ranks row-shard a quantized matrix, each computes
its slice (the CPU oracle stands in for the GPU kernel), the slices are all-gathered, and the result equals
the unsharded GEMV bit for bit.  Also the shard arithmetic for ragged row counts."""
import os
import subprocess
import sys
import textwrap

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_arithmetic(pkg):
    from saient_quartz_b200.shard import shard_bytes, shard_rows
    for n, g in [(4096, 8), (128256, 8), (14336, 4), (1000, 3), (5, 8), (1, 2)]:
        covered = []
        for r in range(g):
            n0, n1, per = shard_rows(n, r, g)
            assert 0 <= n0 <= n1 <= n and n1 - n0 <= per
            covered += list(range(n0, n1))
        assert covered == list(range(n))
    assert shard_rows(28672, 7, 8) == (25088, 28672, 3584)
    b0, b1 = shard_bytes(14, 28672, 8192, 3, 8)
    assert (b1 - b0) == 1024 * (28672 // 256) * 210 and b0 == 3 * (b1 - b0)


WORKER = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, {root!r})
    import numpy as np, torch, torch.distributed as dist
    import __graft_entry__ as entry
    entry.load_package()
    import oracle
    from saient_quartz_b200 import synth
    from saient_quartz_b200.shard import shard_rows, shard_bytes, all_gather_rows
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    ok = True
    for (t, K, N) in [(12, 1024, 77), (14, 2048, 130), (8, 256, 5)]:
        w = synth.make_weights(t, K, N, tensor_id=5)
        x = synth.make_x(K, tensor_id=6)
        n0, n1, per = shard_rows(N, rank, world)
        b0, b1 = shard_bytes(t, K, N, rank, world)
        y_full = torch.zeros(world * per, dtype=torch.float32)
        if n1 > n0:
            y_full[rank * per: rank * per + (n1 - n0)] = torch.from_numpy(oracle.gemv(x, w[b0:b1], t, K, n1 - n0))
        all_gather_rows(y_full, rank, world, per, dist)
        ok &= bool(np.array_equal(y_full[:N].numpy(), oracle.gemv(x, w, t, K, N)))
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)
""")


def test_two_gloo_ranks_shard_and_gather(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)],
                       env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


WINDOW_WORKER = textwrap.dedent("""
    import ctypes as C, os, sys
    sys.path.insert(0, {root!r})
    import numpy as np, torch, torch.distributed as dist
    import __graft_entry__ as entry
    entry.load_package()
    from saient_quartz_b200.shard import PeerWindow, shard_rows

    class FakeLib:
        '''Stands in for the CUDA library: a "window" is a host array, a "handle" names its owner, and the
        exchange itself is carried by gloo, so the host-side protocol (init, handle exchange in rank order,
        attach, push offsets, one wait per exchange) runs without a GPU.'''
        def __init__(self, rank, world):
            self.rank, self.world, self.calls = rank, world, []
            self.window = None
        def quartz_mgpu_handle_bytes(self):
            return 64
        def quartz_mgpu_init(self, rank, world, data_bytes, buf):
            self.window = np.zeros(data_bytes // 4, dtype=np.float32)
            C.memmove(buf, (b"rank%02d" % rank).ljust(64, b"."), 64)
            return 0
        def quartz_mgpu_attach(self, handles):
            self.handles = bytes(handles)
            return 0 if len(self.handles) == 64 * self.world else -1
        def quartz_mgpu_data(self):
            return 1234
        def cuda_gemv_push(self, t, w, x, dst_off, in_dim, rows):
            self.calls.append(("push", dst_off, rows))
        def quartz_mgpu_wait(self):
            self.calls.append(("wait",))
        def quartz_mgpu_fuse_next_wait(self):
            self.calls.append(("fuse",))
        def quartz_mgpu_shutdown(self):
            self.calls.append(("shutdown",))

    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    lib = FakeLib(rank, world)
    win = PeerWindow(lib, rank, world, 4096, dist)
    ok = win.data_ptr == 1234
    # every rank received all handles, in rank order
    ok &= [lib.handles[64 * r:64 * r + 6] for r in range(world)] == [b"rank%02d" % r for r in range(world)]
    N = 1000
    n0, n1, per = shard_rows(N, rank, world)
    win.gemv_push(12, 0, 0, 100 + n0, 4096, n1 - n0)
    win.wait(fused=True)
    win.gemv_push(14, 0, 0, 2000 + n0, 4096, n1 - n0)
    win.wait()
    win.close()
    ok &= lib.calls == [("push", 100 + n0, n1 - n0), ("fuse",), ("push", 2000 + n0, n1 - n0), ("wait",), ("shutdown",)]
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)
""")


def test_two_gloo_ranks_window_protocol(tmp_path):
    """PeerWindow's host side (handle exchange in rank order, attach, push offsets, waits) over gloo with a
    stand-in for the CUDA library."""
    script = tmp_path / "window_worker.py"
    script.write_text(WINDOW_WORKER.format(root=ROOT))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29534", str(script)],
                       env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
