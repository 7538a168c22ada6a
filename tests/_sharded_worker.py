"""Worker for the multi-rank tests: launched once per rank by torchrun.

    BACKEND=gloo : CPU only. The sharding arithmetic (shard_rows, per-shard quantization == slicing the whole,
                   column assembly order) with the CPU oracle standing in for the kernels.
    BACKEND=nccl : one GPU per rank. The CUDA linear on each shard, gathered by NCCL and by the peer gather,
                   against the oracle's result for the whole layer.
Writes "OK <rank>" on success; any assertion fails the process.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch.distributed as dist  # noqa: E402

import oracle  # noqa: E402
from grilly2_b200.sharded import assemble_columns, shard_rows  # noqa: E402


def main() -> None:
    backend = os.environ.get("BACKEND", "gloo")
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if backend == "nccl":
        import torch
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        os.environ["GQ_DEVICE"] = os.environ.get("LOCAL_RANK", str(rank))
        dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank))))
    else:
        dist.init_process_group("gloo")
    rng = np.random.default_rng(2)  # the same on every rank
    n, k, group = 64 * world, 256, 128
    x = rng.standard_normal((3, k)).astype(np.float32)
    w = (rng.standard_normal((n, k)) * 0.015).astype(np.float32)
    b = rng.standard_normal(n).astype(np.float32)
    lo, hi = shard_rows(n, world, rank)
    qf, sf, zf = oracle.quantize_q4(w, group)
    whole = oracle.linear_q4(x, qf, sf, zf, b, k, group)

    # a shard quantizes to exactly the rows of the whole
    qs, ss, zs = oracle.quantize_q4(w[lo:hi], group)
    assert np.array_equal(qs, qf[lo:hi]) and np.array_equal(ss, sf[lo:hi]) and np.array_equal(zs, zf[lo:hi])

    if backend == "gloo":
        mine = oracle.linear_q4(x, qs, ss, zs, b[lo:hi], k, group)
        blocks = [None] * world
        dist.all_gather_object(blocks, mine)
        assert np.array_equal(assemble_columns(blocks), whole)
    else:
        from grilly2_b200 import _C
        from grilly2_b200.sharded import Comm, PeerGather, ShardedLinear
        layer = ShardedLinear.from_full(w, b, world, rank, bits=4, group_size=group)
        assert np.array_equal(layer.q.packed().numpy().view(np.uint32), qf[lo:hi])
        comm = Comm.from_torch_distributed()

        def exchange(obj):
            out = [None] * world
            dist.all_gather_object(out, obj)
            return out

        peers = PeerGather(world, rank, 3, n, exchange)
        for step in range(3):  # several steps: the flag counters and the two buffers must keep working
            xs = (x * (step + 1)).astype(np.float32)
            ref = oracle.linear_q4(xs, qf, sf, zf, b, k, group)
            y_shard = layer.local(_C.Tensor.from_numpy(xs))
            got = comm.all_gather(y_shard).numpy()
            assert np.abs(got - ref).max() / np.abs(ref).max() <= 1e-5, "nccl gather"
            got2 = peers.gather(y_shard).numpy()
            assert np.array_equal(got2, got), "peer gather differs from the nccl gather"
            dist.barrier()
        peers.close()
        # the linear and the gather in one kernel (the ring kernel's shapes), against the oracle on the whole weight
        k2, per = 4096, 80  # 80 features per rank: five 16-row blocks
        w2 = (rng.standard_normal((per * world, k2)) * 0.015).astype(np.float32)
        b2 = rng.standard_normal(per * world).astype(np.float32)
        x2 = rng.standard_normal((3, k2)).astype(np.float32)
        q2, s2, z2 = oracle.quantize_q4(w2, group)
        layer2 = ShardedLinear.from_full(w2, b2, world, rank, bits=4, group_size=group)
        peers2 = PeerGather(world, rank, 3, per * world, exchange)
        for step in range(4):
            xs = (x2 * (step + 1)).astype(np.float32)
            ref = oracle.linear_q4(xs, q2, s2, z2, b2, k2, group)
            got = peers2.linear_gather(layer2.q, _C.Tensor.from_numpy(xs), layer2.bias).numpy()
            assert np.abs(got - ref).max() / np.abs(ref).max() <= 1e-5, f"fused linear + gather, step {step}"
            dist.barrier()
        peers2.close()
        comm.close()
    dist.barrier()
    print(f"OK {rank}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
