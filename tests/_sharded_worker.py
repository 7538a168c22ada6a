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
        from grilly2_b200 import _C, _lib
        from grilly2_b200.sharded import Comm, PeerGather, ShardedLinear
        layer = ShardedLinear.from_full(w, b, world, rank, bits=4, group_size=group)
        assert np.array_equal(layer.q.packed().numpy().view(np.uint32), qf[lo:hi])
        comm = Comm.from_torch_distributed()

        def exchange(obj):
            out = [None] * world
            dist.all_gather_object(out, obj)
            return out

        peers = PeerGather(world, rank, 3, n, exchange)
        for step in range(3):  # several steps: the step word and the two halves of the receive buffer must keep working
            xs = (x * (step + 1)).astype(np.float32)
            ref = oracle.linear_q4(xs, qf, sf, zf, b, k, group)
            y_shard = layer.local(_C.Tensor.from_numpy(xs))
            got = comm.all_gather(y_shard).numpy()
            assert np.abs(got - ref).max() / np.abs(ref).max() <= 1e-5, "nccl gather"
            got2 = peers.gather(y_shard).numpy()
            assert np.array_equal(got2, got), "peer gather differs from the nccl gather"
            dist.barrier()
        peers.close()
        # the linear and the gather in one kernel (the ring kernel's shapes), against the oracle on the whole weight;
        # m = 3 is one pass, m = 8 and m = 16 are passes of four rows
        k2, per = 4096, 80  # 80 features per rank: five blocks of 16 rows
        w2 = (rng.standard_normal((per * world, k2)) * 0.015).astype(np.float32)
        b2 = rng.standard_normal(per * world).astype(np.float32)
        q2, s2, z2 = oracle.quantize_q4(w2, group)
        layer2 = ShardedLinear.from_full(w2, b2, world, rank, bits=4, group_size=group)
        for m2 in (3, 8, 16):
            x2 = rng.standard_normal((m2, k2)).astype(np.float32)
            peers2 = PeerGather(world, rank, m2, per * world, exchange)
            for step in range(4):
                xs = (x2 * (step + 1)).astype(np.float32)
                ref = oracle.linear_q4(xs, q2, s2, z2, b2, k2, group)
                got = peers2.linear_gather(layer2.q, _C.Tensor.from_numpy(xs), layer2.bias).numpy()
                assert np.abs(got - ref).max() / np.abs(ref).max() <= 1e-5, f"fused linear + gather, m = {m2}, step {step}"
                if step == 1:  # the separate gather on the same buffers, in between: one protocol
                    sep = peers2.gather(layer2.q.linear(_C.Tensor.from_numpy(xs), layer2.bias, _lib.KERNEL_RING)).numpy()
                    assert np.array_equal(sep, got), "separate gather differs from the fused one"
                dist.barrier()
            peers2.close()
        # a shard large enough (4 MB and more) for the tcgen05 decode kernel: many rows go through it, the gather adding up its
        # K slices' partial sums as it sends them
        k4, per4 = 8192, 1024
        w4 = (rng.standard_normal((per4 * world, k4)) * 0.015).astype(np.float32)
        b4 = rng.standard_normal(per4 * world).astype(np.float32)
        q4, s4, z4 = oracle.quantize_q4(w4, group)
        layer4 = ShardedLinear.from_full(w4, b4, world, rank, bits=4, group_size=group)
        for m4 in (16, 6):
            peers4 = PeerGather(world, rank, m4, per4 * world, exchange)
            for step in range(3):
                xs = (rng.standard_normal((m4, k4)) * (step + 1)).astype(np.float32)
                ref = oracle.linear_q4(xs, q4, s4, z4, b4, k4, group)
                got = peers4.linear_gather(layer4.q, _C.Tensor.from_numpy(xs), layer4.bias).numpy()
                assert np.abs(got - ref).max() / np.abs(ref).max() <= 1e-5, f"tensor-core linear + gather, m = {m4}, step {step}"
                dist.barrier()
            peers4.close()
        # A captured graph holding ONE gather, replayed many times with a different x each time and no host wait in
        # between: the device alternates the halves of the receive buffer by itself, so a rank that runs ahead never
        # overwrites what a slower one still has to read. Every step's result is kept and checked at the end.
        steps, m3 = 24, 2
        xs_all = rng.standard_normal((steps, m3, k2)).astype(np.float32)
        xs_dev = _C.Tensor.from_numpy(xs_all)
        x_in = _C.Tensor.empty((m3, k2), "float32", persistent=True)
        hist = _C.Tensor.empty((steps, m3, per * world), "float32", persistent=True)
        peers3 = PeerGather(world, rank, m3, per * world, exchange)
        x_in.copy_(xs_dev.narrow_rows(0, 1).reshape((m3, k2)))
        peers3.linear_gather(layer2.q, x_in, layer2.bias)  # eager once
        _C.begin_capture()
        y_cap = peers3.linear_gather(layer2.q, x_in, layer2.bias)
        graph = _C.end_capture()
        _C.synchronize()
        dist.barrier()
        for i in range(steps):
            x_in.copy_(xs_dev.narrow_rows(i, 1).reshape((m3, k2)))
            graph.replay()
            hist.narrow_rows(i, 1).reshape((m3, per * world)).copy_(y_cap)
        got_all = hist.numpy()
        for i in range(steps):
            ref = oracle.linear_q4(xs_all[i], q2, s2, z2, b2, k2, group)
            assert np.abs(got_all[i] - ref).max() / np.abs(ref).max() <= 1e-5, f"replayed gather, step {i}"
        del graph
        dist.barrier()
        peers3.close()
        comm.close()
    dist.barrier()
    print(f"OK {rank}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
