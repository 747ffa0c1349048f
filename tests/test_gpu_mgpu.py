"""Row-sharded GEMV/GEMM with the exchange done by peer stores (cuda_gemv_push / cuda_push_rows /
quartz_mgpu_wait).  One process per GPU; the single-rank case runs on any box, the multi-rank cases
need that many GPUs."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "mgpu_worker.py")


def _gpus():
    import torch
    return torch.cuda.device_count()


def _run(world):
    env = dict(os.environ)
    env["NCCL_NVLS_ENABLE"] = "0"
    if world == 1:
        cmd = [sys.executable, WORKER]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", str(29600 + world), WORKER]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + "\n" + r.stderr[-3000:]
    for k in range(world):
        assert f"rank {k}/{world}: ok" in r.stdout, r.stdout[-3000:]


def test_single_rank_window():
    _run(1)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ranks(world):
    if _gpus() < world:
        pytest.skip(f"needs {world} GPUs")
    _run(world)
