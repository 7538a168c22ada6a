"""Multi-rank tests of the column-sharded linear. The gloo test runs on CPU
(world size 2); the nccl test needs two GPUs and is skipped on a one-GPU box."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "_sharded_worker.py")


def run_ranks(world: int, backend: str, port: int) -> str:
    env = dict(os.environ, BACKEND=backend, OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), WORKER]
    p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    return p.stdout


def test_shard_rows_and_assembly():
    import numpy as np
    from grilly2_b200.sharded import assemble_columns, shard_rows
    assert [shard_rows(28672, 8, r) for r in (0, 7)] == [(0, 3584), (25088, 28672)]
    with pytest.raises(ValueError, match="does not divide"):
        shard_rows(10, 4, 0)
    with pytest.raises(ValueError, match="out of range"):
        shard_rows(8, 2, 2)
    a, b = np.ones((2, 3)), np.zeros((2, 3))
    assert assemble_columns([a, b]).shape == (2, 6) and assemble_columns([a, b])[0, 3] == 0


def test_sharding_over_two_gloo_ranks_on_cpu():
    out = run_ranks(2, "gloo", 29541)
    assert "OK 0" in out and "OK 1" in out


@pytest.mark.gpu
def test_sharded_linear_over_two_gpus():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = run_ranks(2, "nccl", 29542)
    assert "OK 0" in out and "OK 1" in out
