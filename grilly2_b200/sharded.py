"""Column-sharded quantized linear over the GPUs of one box (one process per
GPU). The reference runs on a single device; this is the multi-GPU form of its
linear: rank r owns output features ``[r n / W, (r + 1) n / W)``, quantizes and
multiplies its own rows (exactly what the whole weight would give, because the
parameters are per row / per (row, group)), and the blocks of ``y`` are
gathered so that every rank holds ``y[m][n]``.

Two gathers are offered: NCCL (``Comm`` + ``all_gather``) and this library's
own collective over peer-mapped memory (``PeerGather``: one 64-bit
value-and-step word per output, no fence or signal).
Rendezvous data (the NCCL id, the IPC handles) travels through whatever the
caller has; ``from_torch_distributed`` helpers use ``torch.distributed``'s
object collectives, which work on gloo and nccl alike.
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import _C, _lib
from ._lib import check


def shard_rows(n: int, world: int, rank: int) -> tuple[int, int]:
    """The output features rank ``rank`` of ``world`` owns: equal contiguous blocks."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} of {world} is out of range")
    if n % world:
        raise ValueError(f"out_features = {n} does not divide over {world} ranks")
    per = n // world
    return rank * per, (rank + 1) * per


def assemble_columns(blocks) -> np.ndarray:
    """What a gather must produce, on the host: rank blocks ``[m, n / W]`` side by side."""
    return np.concatenate([np.asarray(b) for b in blocks], axis=1)


class Comm:
    """An NCCL communicator owned by the backend context."""

    def __init__(self, world: int, rank: int, unique_id: bytes) -> None:
        out = ctypes.c_void_p()
        buf = ctypes.create_string_buffer(unique_id, 128)
        check(_lib.load().gq_comm_create(_C.context(), world, rank, buf, ctypes.byref(out)))
        self._c, self.world, self.rank = out, world, rank

    @staticmethod
    def new_id() -> bytes:
        buf = ctypes.create_string_buffer(128)
        check(_lib.load().gq_comm_unique_id(buf, 128))
        return buf.raw

    @classmethod
    def from_torch_distributed(cls) -> "Comm":
        import torch.distributed as dist
        box = [cls.new_id() if dist.get_rank() == 0 else None]
        dist.broadcast_object_list(box, src=0)
        return cls(dist.get_world_size(), dist.get_rank(), box[0])

    def all_gather(self, y_shard: "_C.Tensor", out: "_C.Tensor | None" = None) -> "_C.Tensor":
        m = y_shard.numel() // y_shard.shape[-1] if y_shard.shape[-1] else 0
        n_shard = y_shard.shape[-1]
        if out is None:
            out = _C.Tensor.empty(y_shard.shape[:-1] + (n_shard * self.world,), "float32")
        check(_lib.load().gq_all_gather_columns(_C.context(), self._c, y_shard.storage.handle, out.storage.handle, m, n_shard))
        return out

    def close(self) -> None:
        if self._c:
            _lib.load().gq_comm_destroy(_C.context(), self._c)
            self._c = None


class PeerGather:
    """This library's own gather over CUDA IPC for a fixed (m, n_full). Holds this rank's receive buffer (two halves that
    the DEVICE alternates by step parity, so a captured call alternates by itself at every replay), its two state words,
    and handles to every other rank's receive buffer. ``gather`` and ``linear_gather`` speak the same protocol and may be
    mixed; every rank must make the same sequence of calls."""

    def __init__(self, world: int, rank: int, m: int, n_full: int, exchange) -> None:
        """``exchange(obj) -> list`` returns every rank's ``obj`` in rank order
        (e.g. ``torch.distributed.all_gather_object``)."""
        lib, ctx = _lib.load(), _C.context()
        self.world, self.rank, self.m, self.n_full = world, rank, m, n_full
        self.recv = _C.Tensor.from_numpy(np.zeros(2 * m * n_full * 2, dtype=np.int32), persistent=True)  # 64-bit words
        self.state = _C.Tensor.from_numpy(np.zeros(2, dtype=np.int32), persistent=True)
        _C.synchronize()
        buf = ctypes.create_string_buffer(64)
        check(lib.gq_buffer_ipc_export(ctx, self.recv.storage.handle, buf, 64))
        everyone = exchange(buf.raw)
        self._opened = []

        def open_(raw):
            out = ctypes.c_uint64()
            check(lib.gq_buffer_ipc_open(ctx, ctypes.create_string_buffer(raw, 64), 2 * m * n_full * 8, ctypes.byref(out)))
            self._opened.append(out.value)
            return out.value

        self._recv_handles = [self.recv.storage.handle if r == rank else open_(everyone[r]) for r in range(world)]

    def _out(self, out):
        return out if out is not None else _C.Tensor.empty((self.m, self.n_full), "float32")

    def gather(self, y_shard: "_C.Tensor", out: "_C.Tensor | None" = None) -> "_C.Tensor":
        lib, ctx = _lib.load(), _C.context()
        arr = ctypes.c_uint64 * self.world
        m = y_shard.numel() // y_shard.shape[-1]
        if m != self.m or y_shard.shape[-1] * self.world != self.n_full:
            raise RuntimeError(f"gather: a block of {m} x {y_shard.shape[-1]} over {self.world} ranks does not fill y_full {self.m} x {self.n_full}")
        out = self._out(out)
        check(lib.gq_peer_gather(ctx, y_shard.storage.handle, m, y_shard.shape[-1], self.rank, self.world, arr(*self._recv_handles),
                                 self.state.storage.handle, out.storage.handle))
        return out

    def linear_gather(self, weight: "_C.Int4Weight", x: "_C.Tensor", bias: "_C.Tensor | None" = None,
                      out: "_C.Tensor | None" = None) -> "_C.Tensor":
        """This rank's int4 block times x, sent from the GEMV's epilogue to every rank: one kernel for the linear and the
        gather (group size 128, in_features 4096 or 8192, up to 16 rows of x)."""
        lib, ctx = _lib.load(), _C.context()
        arr = ctypes.c_uint64 * self.world
        n_shard, k = weight.shape
        m = x.numel() // k
        if m != self.m or n_shard * self.world != self.n_full:
            raise RuntimeError(f"linear_gather: {m} x {n_shard} x {self.world} ranks does not fill y_full {self.m} x {self.n_full}")
        out = self._out(out)
        check(lib.gq_int4_linear_gather(ctx, x.storage.handle, x.offset, m, k, weight._qt.storage.handle, weight._scale.storage.handle,
                                        weight._zero.storage.handle, bias.storage.handle if bias is not None else 0,
                                        bias.offset if bias is not None else 0, n_shard, weight._group, self.rank, self.world,
                                        arr(*self._recv_handles), self.state.storage.handle, out.storage.handle))
        return out

    def close(self) -> None:
        lib, ctx = _lib.load(), _C.context()
        _C.synchronize()
        for h in self._opened:
            lib.gq_buffer_release(ctx, h)
        self._opened = []


class ShardedLinear:
    """This rank's block of a quantized linear plus the gather of its output."""

    def __init__(self, weight_rows: np.ndarray, bias_rows, world: int, rank: int, bits: int = 4, group_size: int = 128) -> None:
        w = _C.Tensor.from_numpy(np.ascontiguousarray(weight_rows, dtype=np.float32))
        self.q = _C.Int4Weight.quantize(w, group_size) if bits == 4 else _C.Int8Weight.quantize(w)
        self.bias = None if bias_rows is None else _C.Tensor.from_numpy(np.ascontiguousarray(bias_rows, dtype=np.float32), persistent=True)
        self.world, self.rank = world, rank

    @classmethod
    def from_full(cls, weight: np.ndarray, bias, world: int, rank: int, **kw) -> "ShardedLinear":
        lo, hi = shard_rows(weight.shape[0], world, rank)
        return cls(weight[lo:hi], None if bias is None else bias[lo:hi], world, rank, **kw)

    def local(self, x: "_C.Tensor") -> "_C.Tensor":
        return self.q.linear(x, self.bias)
