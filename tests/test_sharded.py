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
@pytest.mark.parametrize("m,n,k", [(1, 80, 4096), (3, 333, 4096), (2, 48, 8192), (4, 5, 4096), (9, 100, 4096), (16, 37, 8192)])
def test_fused_linear_gather_with_a_single_rank_equals_the_linear(m, n, k):
    """World size 1 (the only peer is the rank itself): gq_int4_linear_gather must equal gq_int4_linear on the same (ring)
    kernel, step after step."""
    import numpy as np
    from grilly2_b200 import _C, _lib
    from grilly2_b200.sharded import PeerGather
    rng = np.random.default_rng(n + k)
    w = _C.Int4Weight.quantize(_C.Tensor.from_numpy((rng.standard_normal((n, k)) * 0.02).astype(np.float32)), 128)
    bias = _C.Tensor.from_numpy(rng.standard_normal(n).astype(np.float32))
    peers = PeerGather(1, 0, m, n, lambda obj: [obj])
    for step in range(3):
        x = _C.Tensor.from_numpy(rng.standard_normal((m, k)).astype(np.float32))
        want = w.linear(x, bias, _lib.KERNEL_RING).numpy()
        got = peers.linear_gather(w, x, bias).numpy()
        np.testing.assert_array_equal(got, want)
    peers.close()


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k", [(16, 1024, 8192), (9, 2304, 4096), (8, 1100, 12288)])
def test_many_rows_on_a_large_shard_take_the_tensor_core_route_and_equal_the_linear(m, n, k):
    """Five and more rows on a weight of 4 MB and more: gq_int4_linear_gather runs the tcgen05 decode kernel and lets the
    gather add up its K slices; with one rank that must equal gq_int4_linear (which picks the same kernel and adds the
    slices in the same order) bit for bit, and the CPU oracle within 1e-5, step after step."""
    import numpy as np
    import oracle
    from grilly2_b200 import _C
    from grilly2_b200.sharded import PeerGather
    rng = np.random.default_rng(n + k)
    wf = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    w = _C.Int4Weight.quantize(_C.Tensor.from_numpy(wf), 128)
    q, s, z = oracle.quantize_q4(wf, 128)
    b = rng.standard_normal(n).astype(np.float32)
    bias = _C.Tensor.from_numpy(b)
    peers = PeerGather(1, 0, m, n, lambda obj: [obj])
    for step in range(3):
        xs = rng.standard_normal((m, k)).astype(np.float32)
        x = _C.Tensor.from_numpy(xs)
        want = w.linear(x, bias).numpy()
        got = peers.linear_gather(w, x, bias).numpy()
        np.testing.assert_array_equal(got, want)
        ref = oracle.linear_q4(xs, q, s, z, b, k, 128)
        assert np.abs(got - ref).max() / np.abs(ref).max() <= 1e-5
    peers.close()


@pytest.mark.gpu
@pytest.mark.parametrize("fused", [False, True], ids=["gather", "linear_gather"])
def test_a_gather_whose_peer_never_sends_gives_up_and_reports_the_rank(fused):
    """Failure detection without a fault: two "ranks" whose receive buffers both live in this process, and nobody
    plays rank 1. With the wait limit at 20 ms the kernel returns, the next host wait is GQ_ERR naming rank 1, the
    status clears, and an ordinary linear on the same context then answers correctly."""
    import ctypes

    import numpy as np

    import oracle
    from grilly2_b200 import _C, _lib
    lib, ctx = _lib.load(), _C.context()
    rng = np.random.default_rng(5)
    m, n_shard, k = 2, 48, 4096
    w = (rng.standard_normal((n_shard, k)) * 0.02).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    wt = _C.Int4Weight.quantize(_C.Tensor.from_numpy(w), 128)
    xt = _C.Tensor.from_numpy(x)
    recv = [_C.Tensor.from_numpy(np.zeros(2 * m * 2 * n_shard * 2, dtype=np.int32), persistent=True) for _ in range(2)]
    state = _C.Tensor.from_numpy(np.zeros(2, dtype=np.int32), persistent=True)
    y_full = _C.Tensor.empty((m, 2 * n_shard), "float32")
    handles = (ctypes.c_uint64 * 2)(recv[0].storage.handle, recv[1].storage.handle)
    _C.synchronize()
    _lib.check(lib.gq_set_wait_limit_us(ctx, 20000))
    try:
        if fused:
            _lib.check(lib.gq_int4_linear_gather(ctx, xt.storage.handle, 0, m, k, wt._qt.storage.handle, wt._scale.storage.handle,
                                                 wt._zero.storage.handle, 0, 0, n_shard, 128, 0, 2, handles, state.storage.handle,
                                                 y_full.storage.handle))
        else:
            y = wt.linear(xt)
            _lib.check(lib.gq_peer_gather(ctx, y.storage.handle, m, n_shard, 0, 2, handles, state.storage.handle, y_full.storage.handle))
        assert lib.gq_synchronize(ctx) == _lib.GQ_ERR
        assert "rank 1" in _lib.last_error() and "17" in _lib.last_error()
        assert lib.gq_synchronize(ctx) == _lib.GQ_OK  # reported once; the context stays usable
    finally:
        _lib.check(lib.gq_set_wait_limit_us(ctx, 0))
    # this rank's own half did arrive
    q, sc, z = oracle.quantize_q4(w, 128)
    ref = oracle.linear_q4(x, q, sc, z, None, k, 128)
    got = y_full.numpy()[:, :n_shard]
    assert np.abs(got - ref).max() / np.abs(ref).max() <= 1e-5
    assert np.abs(wt.linear(xt).numpy() - ref).max() / np.abs(ref).max() <= 1e-5
