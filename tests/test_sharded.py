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


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k", [(1, 80, 4096), (3, 333, 4096), (2, 48, 8192), (4, 5, 4096)])
def test_fused_linear_gather_with_a_single_rank_equals_the_linear(m, n, k):
    """World size 1 (the only peer is the rank itself): gq_int4_linear_gather must equal gq_int4_linear, step after step."""
    import numpy as np
    from grilly2_b200 import _C
    from grilly2_b200.sharded import PeerGather
    rng = np.random.default_rng(n + k)
    w = _C.Int4Weight.quantize(_C.Tensor.from_numpy((rng.standard_normal((n, k)) * 0.02).astype(np.float32)), 128)
    bias = _C.Tensor.from_numpy(rng.standard_normal(n).astype(np.float32))
    peers = PeerGather(1, 0, m, n, lambda obj: [obj])
    for step in range(3):
        x = _C.Tensor.from_numpy(rng.standard_normal((m, k)).astype(np.float32))
        want = w.linear(x, bias).numpy()
        got = peers.linear_gather(w, x, bias).numpy()
        np.testing.assert_array_equal(got, want)
    peers.close()
