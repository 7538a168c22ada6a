"""The compiled core as Python sees it: the stand-in for the reference's PyO3
module ``grilly._C`` (crates/grilly-py/src/infer.rs:82-239 for the quantized
weights, crates/grilly-py/src/ops.rs:484,584,611-657 for capture and
statistics) and for the Rust types behind it
(crates/grilly-infer/src/quant.rs:86-305, quant4.rs:71-443). Same class and
method names, same argument meaning, same refusals; underneath, every method
is a call into the C ABI of include/gq.h.
"""
from __future__ import annotations

import ctypes
import threading

import numpy as np

from . import _lib
from ._lib import KERNEL_AUTO, MEM_DEVICE, MEM_PERSISTENT, check

F32, I32 = "float32", "int32"
_NP = {F32: np.float32, I32: np.int32}

_ctx = None
_ctx_lock = threading.Lock()


def context():
    """The process-wide context on cuda:0 (the reference has one default
    device, crates/grilly-core/src/device.rs:261-269). GQ_DEVICE picks another
    ordinal, for one process per GPU."""
    global _ctx
    if _ctx is None:
        with _ctx_lock:
            if _ctx is None:
                import os
                lib = _lib.load()
                out = ctypes.c_void_p()
                check(lib.gq_create(int(os.environ.get("GQ_DEVICE", os.environ.get("LOCAL_RANK", "0"))), ctypes.byref(out)))
                _ctx = out
    return _ctx


def _l():
    return _lib.load()


class _Storage:
    """One gq_buf handle, released when the last tensor naming it dies."""

    __slots__ = ("handle", "bytes", "parent", "__weakref__")

    def __init__(self, nbytes: int, mem: int) -> None:
        out = ctypes.c_uint64()
        check(_l().gq_buffer_create(context(), int(nbytes), mem, ctypes.byref(out)))
        self.handle, self.bytes, self.parent = out.value, int(nbytes), None

    @classmethod
    def window(cls, parent: "_Storage", byte_offset: int, nbytes: int) -> "_Storage":
        """A handle of its own onto ``nbytes`` of ``parent`` from ``byte_offset`` on (gq_buffer_wrap of the parent's
        address): for operators that write their output at the start of the buffer they are given, so that several
        outputs can land side by side in one allocation. The parent stays alive as long as the window does."""
        if byte_offset < 0 or nbytes < 0 or byte_offset + nbytes > parent.bytes or byte_offset % 16:
            raise IndexError("window out of range (or not 16-byte aligned)")
        ptr, out = ctypes.c_void_p(), ctypes.c_uint64()
        check(_l().gq_buffer_ptr(context(), parent.handle, ctypes.byref(ptr)))
        check(_l().gq_buffer_wrap(context(), ctypes.c_void_p(ptr.value + byte_offset), int(nbytes), ctypes.byref(out)))
        self = object.__new__(cls)
        self.handle, self.bytes, self.parent = out.value, int(nbytes), parent
        return self

    def __del__(self) -> None:
        try:
            if self.handle and _ctx is not None:
                _l().gq_buffer_release(_ctx, self.handle)
        except Exception:  # interpreter shutdown
            pass
        self.handle = 0


class Tensor:
    """A contiguous row-major run of float32 or int32 in a device buffer,
    located by an element offset (crates/grilly-core/src/tensor.rs:10-30)."""

    __slots__ = ("storage", "shape", "dtype", "offset")

    def __init__(self, storage: _Storage, shape, dtype: str, offset: int = 0) -> None:
        self.storage, self.shape, self.dtype, self.offset = storage, tuple(int(s) for s in shape), dtype, int(offset)

    @staticmethod
    def empty(shape, dtype: str = F32, persistent: bool = False) -> "Tensor":
        shape = tuple(int(s) for s in shape)
        n = int(np.prod(shape, dtype=np.int64)) if shape else 1
        return Tensor(_Storage(n * 4, MEM_PERSISTENT if persistent else MEM_DEVICE), shape, dtype)

    @staticmethod
    def from_numpy(a, persistent: bool = False) -> "Tensor":
        a = np.asarray(a)
        if a.dtype == np.float32:
            dtype = F32
        elif a.dtype == np.int32:
            dtype = I32
        else:
            raise NotImplementedError(f"grilly: dtype {a.dtype} is not implemented yet (this backend has float32 and int32)")
        a = np.ascontiguousarray(a)
        t = Tensor.empty(a.shape, dtype, persistent)
        if a.size:
            check(_l().gq_upload(context(), t.storage.handle, 0, a.ctypes.data_as(ctypes.c_void_p), a.nbytes))
        return t

    def numel(self) -> int:
        return int(np.prod(self.shape, dtype=np.int64)) if self.shape else 1

    def numpy(self) -> np.ndarray:
        out = np.empty(self.shape, dtype=_NP[self.dtype])
        check(_l().gq_download(context(), self.storage.handle, self.offset * 4,
                               out.ctypes.data_as(ctypes.c_void_p), out.nbytes))
        return out

    def reshape(self, shape) -> "Tensor":
        shape = tuple(int(s) for s in shape)
        if int(np.prod(shape, dtype=np.int64)) != self.numel():
            raise RuntimeError(f"shape {shape} is invalid for input of size {self.numel()}")
        return Tensor(self.storage, shape, self.dtype, self.offset)

    def narrow_rows(self, start: int, length: int) -> "Tensor":
        """Rows [start, start + length) of the leading dimension: still
        contiguous, so a view at an element offset."""
        inner = self.numel() // self.shape[0] if self.shape[0] else 0
        if start < 0 or length < 0 or start + length > self.shape[0]:
            raise IndexError("index out of range in self")
        return Tensor(self.storage, (length,) + self.shape[1:], self.dtype, self.offset + start * inner)

    def window_rows(self, start: int, length: int) -> "Tensor":
        """Rows [start, start + length) as a tensor at offset 0 of a buffer handle of its own (see _Storage.window)."""
        inner = self.numel() // self.shape[0] if self.shape[0] else 0
        if start < 0 or length < 0 or start + length > self.shape[0]:
            raise IndexError("index out of range in self")
        st = _Storage.window(self.storage, (self.offset + start * inner) * 4, length * inner * 4)
        return Tensor(st, (length,) + self.shape[1:], self.dtype, 0)

    def clone_data(self) -> "Tensor":
        out = Tensor.empty(self.shape, self.dtype)
        out.copy_(self)
        return out

    def copy_(self, src: "Tensor") -> "Tensor":
        if src.shape != self.shape or src.dtype != self.dtype:
            raise RuntimeError(f"copy_: {src.shape} {src.dtype} does not match {self.shape} {self.dtype}")
        if self.numel():
            check(_l().gq_copy(context(), src.storage.handle, src.offset * 4, self.storage.handle, self.offset * 4,
                               self.numel() * 4))
        return self


def _require(t, dtype, what):
    if not isinstance(t, Tensor):
        raise TypeError(f"{what} must be a tensor, got {type(t).__name__}")
    if t.dtype != dtype:
        # crates/grilly-core: require_float -> Error::NotImplemented
        raise NotImplementedError(f"grilly: {what} with dtype {t.dtype} is not implemented yet (expected {dtype})")
    return t


def _words8(k: int) -> int:
    return -(-k // 16) * 4


def _words4(k: int) -> int:
    return -(-k // 32) * 4


def _check_linear(kind, input, bias, n, k):
    _require(input, F32, "linear")
    if not input.shape or input.shape[-1] != k:
        raise RuntimeError(f"linear: input {list(input.shape)} does not end in in_features = {k}")
    if bias is not None:
        _require(bias, F32, "linear")
        if bias.shape != (n,):
            raise RuntimeError(f"linear: bias must be ({n},), got {list(bias.shape)}")
    out_shape = input.shape[:-1] + (n,)
    m = input.numel() // max(k, 1)
    return out_shape, m


def _check_grad(kind, grad, n):
    _require(grad, F32, "linear backward")
    if not grad.shape or grad.shape[-1] != n:
        raise RuntimeError(f"linear backward: grad {list(grad.shape)} does not end in out_features = {n}")
    return grad.numel() // max(n, 1)


def _output(out, shape):
    """A fresh output, or the caller's: float32, the right size, at the start of its buffer (the operators write there)."""
    if out is None:
        return Tensor.empty(shape, F32)
    _require(out, F32, "linear output")
    if out.numel() != int(np.prod(shape, dtype=np.int64)) or out.offset:
        raise RuntimeError(f"linear: the output must hold {list(shape)} at offset 0 of its buffer, got {list(out.shape)} at {out.offset}")
    return out


class Int8Weight:
    """A linear layer's weight, int8 per output row with a float32 scale, in
    persistent device memory (crates/grilly-infer/src/quant.rs:84-94)."""

    __slots__ = ("_qt", "_scale", "_shape")

    def __init__(self, q: Tensor, scale: Tensor, shape) -> None:
        self._qt, self._scale, self._shape = q, scale, tuple(shape)

    @staticmethod
    def quantize(weight: Tensor) -> "Int8Weight":
        _require(weight, F32, "int8 weight-only quantization")
        if len(weight.shape) != 2:
            raise RuntimeError(f"expected a 2-D weight (out_features, in_features), got {list(weight.shape)}")
        n, k = weight.shape
        if k == 0:
            raise RuntimeError("cannot quantize a weight with no input features")
        q = Tensor.empty((n, _words8(k)), I32, persistent=True)
        scale = Tensor.empty((n,), F32, persistent=True)
        check(_l().gq_int8_quantize(context(), weight.storage.handle, weight.offset, n, k, q.storage.handle,
                                    scale.storage.handle))
        return Int8Weight(q, scale, (n, k))

    @staticmethod
    def quantize_fused(weights) -> "Int8Weight":
        """The float32 parts of a fused projection (same in_features), quantized straight into ONE weight at their row
        offsets: equal bit for bit to ``cat`` of the parts quantized apart, without ever holding the parts twice."""
        weights = list(weights)
        if not weights:
            raise RuntimeError("Int8Weight::quantize_fused: no weights")
        for w in weights:
            _require(w, F32, "int8 weight-only quantization")
            if len(w.shape) != 2:
                raise RuntimeError(f"expected a 2-D weight (out_features, in_features), got {list(w.shape)}")
        k = weights[0].shape[1]
        if k == 0 or any(w.shape[1] != k for w in weights):
            raise RuntimeError(f"Int8Weight::quantize_fused: in_features differ or are zero ({[w.shape[1] for w in weights]})")
        n = sum(w.shape[0] for w in weights)
        q = Tensor.empty((n, _words8(k)), I32, persistent=True)
        scale = Tensor.empty((n,), F32, persistent=True)
        row = 0
        for w in weights:
            check(_l().gq_int8_quantize_rows(context(), w.storage.handle, w.offset, w.shape[0], k, q.storage.handle, scale.storage.handle,
                                             row, n))
            row += w.shape[0]
        return Int8Weight(q, scale, (n, k))

    @staticmethod
    def cat(parts) -> "Int8Weight":
        parts = list(parts)
        if not parts:
            raise RuntimeError("Int8Weight::cat: no weights")
        k = parts[0]._shape[1]
        if any(p._shape[1] != k for p in parts):
            raise RuntimeError(f"Int8Weight::cat: in_features differ ({[p._shape[1] for p in parts]})")
        n = sum(p._shape[0] for p in parts)
        words = _words8(k)
        q = Tensor.empty((n, words), I32, persistent=True)
        scale = Tensor.empty((n,), F32, persistent=True)
        row = 0
        for p in parts:
            q.narrow_rows(row, p._shape[0]).copy_(p._qt)
            scale.narrow_rows(row, p._shape[0]).copy_(p._scale)
            row += p._shape[0]
        return Int8Weight(q, scale, (n, k))

    @property
    def shape(self):
        return self._shape

    @property
    def nbytes(self) -> int:
        return self._qt.numel() * 4 + self._scale.numel() * 4

    def scale(self) -> Tensor:
        return self._scale

    def packed(self) -> Tensor:
        """The (out_features, words) int32 tensor itself (no counterpart in
        the PyO3 class, where it stays private: exposed for the sharded and
        benchmark callers in this package)."""
        return self._qt

    def qdata(self) -> bytes:
        """The int8 values, row-major (out_features, in_features), padding stripped."""
        n, k = self._shape
        raw = self._qt.numpy().view(np.int8).reshape(n, -1)
        return raw[:, :k].tobytes()

    def dequantize(self) -> Tensor:
        n, k = self._shape
        w = Tensor.empty((n, k), F32)
        check(_l().gq_int8_dequantize(context(), self._qt.storage.handle, self._scale.storage.handle, n, k,
                                      w.storage.handle))
        return w

    def linear(self, input: Tensor, bias: Tensor | None = None, kernel: int = KERNEL_AUTO, out: Tensor | None = None) -> Tensor:
        n, k = self._shape
        out_shape, m = _check_linear("int8", input, bias, n, k)
        y = _output(out, out_shape)
        check(_l().gq_int8_linear(context(), input.storage.handle, input.offset, m, k, self._qt.storage.handle,
                                  self._scale.storage.handle, bias.storage.handle if bias is not None else 0,
                                  bias.offset if bias is not None else 0, n, y.storage.handle, kernel))
        return y

    def linear_backward(self, grad: Tensor, need_input: bool = True, need_bias: bool = False):
        """(grad_input, grad_bias) of ``linear`` with the weight frozen: grad @ dequantize(W) and grad summed over the
        leading dimensions (crates/grilly-infer/src/quant.rs:326-349). The weight itself gets no gradient."""
        n, k = self._shape
        m = _check_grad("int8", grad, n)
        gx = Tensor.empty(tuple(grad.shape[:-1]) + (k,), F32) if need_input else None
        gb = Tensor.empty((n,), F32) if need_bias else None
        check(_l().gq_int8_linear_backward(context(), grad.storage.handle, grad.offset, m, self._qt.storage.handle,
                                           self._scale.storage.handle, n, k, gx.storage.handle if gx is not None else 0,
                                           gb.storage.handle if gb is not None else 0))
        return gx, gb

    def linear_norm(self, x: Tensor, residual: Tensor | None, norm_weight: Tensor, eps: float, bias: Tensor | None = None,
                    want_sum: bool = False):
        """One row: h = x + residual; returns (W . rms_norm(h) * norm_weight + bias, h if want_sum else None) in one launch."""
        n, k = self._shape
        if x.numel() != k or x.offset or (residual is not None and (residual.numel() != k or residual.offset)):
            raise RuntimeError(f"linear_norm takes one row of {k} values at offset 0")
        y = Tensor.empty((1, n), F32)
        h = Tensor.empty((1, k), F32) if want_sum else None
        check(_l().gq_int8_linear_norm(context(), x.storage.handle, residual.storage.handle if residual is not None else 0,
                                       norm_weight.storage.handle, eps, h.storage.handle if h is not None else 0, k,
                                       self._qt.storage.handle, self._scale.storage.handle,
                                       bias.storage.handle if bias is not None else 0, bias.offset if bias is not None else 0, n,
                                       y.storage.handle))
        return y, h

    def linear_swiglu(self, gate_up: Tensor, bias: Tensor | None = None) -> Tensor:
        """One row of gate | up (2 k values): W . (silu(gate) * up) + bias in one launch."""
        n, k = self._shape
        if gate_up.numel() != 2 * k or gate_up.offset:
            raise RuntimeError(f"linear_swiglu takes one row of {2 * k} values at offset 0")
        y = Tensor.empty((1, n), F32)
        check(_l().gq_int8_linear_swiglu(context(), gate_up.storage.handle, k, self._qt.storage.handle, self._scale.storage.handle,
                                         bias.storage.handle if bias is not None else 0, bias.offset if bias is not None else 0, n,
                                         y.storage.handle))
        return y


class Int4Weight:
    """A linear layer's weight, int4 with a float32 scale and zero point per
    group, in persistent device memory (crates/grilly-infer/src/quant4.rs:69-81)."""

    __slots__ = ("_qt", "_scale", "_zero", "_shape", "_group")

    def __init__(self, q, scale, zero, shape, group) -> None:
        self._qt, self._scale, self._zero, self._shape, self._group = q, scale, zero, tuple(shape), int(group)

    @staticmethod
    def _check_group(group_size) -> None:
        if group_size <= 0 or group_size % 32:
            raise RuntimeError(f"int4 group_size must be a positive multiple of 32, got {group_size}")

    @staticmethod
    def quantize(weight: Tensor, group_size: int) -> "Int4Weight":
        _require(weight, F32, "int4 weight-only quantization")
        if len(weight.shape) != 2:
            raise RuntimeError(f"expected a 2-D weight (out_features, in_features), got {list(weight.shape)}")
        n, k = weight.shape
        if k == 0:
            raise RuntimeError("cannot quantize a weight with no input features")
        Int4Weight._check_group(group_size)
        groups = -(-k // group_size)
        q = Tensor.empty((n, _words4(k)), I32, persistent=True)
        scale = Tensor.empty((n, groups), F32, persistent=True)
        zero = Tensor.empty((n, groups), F32, persistent=True)
        check(_l().gq_int4_quantize(context(), weight.storage.handle, weight.offset, n, k, group_size,
                                    q.storage.handle, scale.storage.handle, zero.storage.handle))
        return Int4Weight(q, scale, zero, (n, k), group_size)

    @staticmethod
    def from_parts(q: Tensor, scale: Tensor, zero: Tensor, in_features: int, group_size: int) -> "Int4Weight":
        Int4Weight._check_group(group_size)
        if len(q.shape) != 2:
            raise RuntimeError(f"expected packed levels (out_features, words), got {list(q.shape)}")
        n, words = q.shape
        groups = -(-in_features // group_size)
        if words != _words4(in_features):
            raise RuntimeError(f"packed levels must be {_words4(in_features)} words per row for in_features "
                               f"{in_features}, got {words}")
        if scale.shape != (n, groups) or zero.shape != (n, groups):
            raise RuntimeError(f"scale and zero must be ({n}, {groups}), got {list(scale.shape)} and {list(zero.shape)}")
        if q.dtype != I32:
            raise RuntimeError(f"packed levels must be int32 words, got {q.dtype}")
        _require(scale, F32, "int4 weight")
        _require(zero, F32, "int4 weight")

        def held(src, dtype):
            out = Tensor.empty(src.shape, dtype, persistent=True)
            out.copy_(src)
            return out

        return Int4Weight(held(q, I32), held(scale, F32), held(zero, F32), (n, in_features), group_size)

    @staticmethod
    def quantize_fused(weights, group_size: int) -> "Int4Weight":
        """As Int8Weight.quantize_fused: the parts quantized straight into one weight at their row offsets."""
        weights = list(weights)
        if not weights:
            raise RuntimeError("Int4Weight::quantize_fused: no weights")
        Int4Weight._check_group(group_size)
        for w in weights:
            _require(w, F32, "int4 weight-only quantization")
            if len(w.shape) != 2:
                raise RuntimeError(f"expected a 2-D weight (out_features, in_features), got {list(w.shape)}")
        k = weights[0].shape[1]
        if k == 0 or any(w.shape[1] != k for w in weights):
            raise RuntimeError(f"Int4Weight::quantize_fused: in_features differ or are zero ({[w.shape[1] for w in weights]})")
        n, groups = sum(w.shape[0] for w in weights), -(-k // group_size)
        q = Tensor.empty((n, _words4(k)), I32, persistent=True)
        scale = Tensor.empty((n, groups), F32, persistent=True)
        zero = Tensor.empty((n, groups), F32, persistent=True)
        row = 0
        for w in weights:
            check(_l().gq_int4_quantize_rows(context(), w.storage.handle, w.offset, w.shape[0], k, group_size, q.storage.handle,
                                             scale.storage.handle, zero.storage.handle, row, n))
            row += w.shape[0]
        return Int4Weight(q, scale, zero, (n, k), group_size)

    @staticmethod
    def cat(parts) -> "Int4Weight":
        parts = list(parts)
        if not parts:
            raise RuntimeError("Int4Weight::cat: no weights")
        k, group = parts[0]._shape[1], parts[0]._group
        if any(p._shape[1] != k for p in parts):
            raise RuntimeError(f"Int4Weight::cat: in_features differ ({[p._shape[1] for p in parts]})")
        if any(p._group != group for p in parts):
            raise RuntimeError(f"Int4Weight::cat: group sizes differ ({[p._group for p in parts]})")
        n = sum(p._shape[0] for p in parts)
        groups = -(-k // group)
        q = Tensor.empty((n, _words4(k)), I32, persistent=True)
        scale = Tensor.empty((n, groups), F32, persistent=True)
        zero = Tensor.empty((n, groups), F32, persistent=True)
        row = 0
        for p in parts:
            q.narrow_rows(row, p._shape[0]).copy_(p._qt)
            scale.narrow_rows(row, p._shape[0]).copy_(p._scale)
            zero.narrow_rows(row, p._shape[0]).copy_(p._zero)
            row += p._shape[0]
        return Int4Weight(q, scale, zero, (n, k), group)

    @property
    def shape(self):
        return self._shape

    @property
    def group_size(self) -> int:
        return self._group

    @property
    def nbytes(self) -> int:
        return (self._qt.numel() + self._scale.numel() + self._zero.numel()) * 4

    def scale(self) -> Tensor:
        return self._scale

    def zero(self) -> Tensor:
        return self._zero

    def packed(self) -> Tensor:
        return self._qt

    def qdata(self) -> bytes:
        """The packed levels: ceil(in_features / 2) bytes per row, the earlier
        value in the low nibble."""
        n, k = self._shape
        raw = self._qt.numpy().view(np.uint8).reshape(n, -1)
        return raw[:, :-(-k // 2)].tobytes()

    def dequantize(self) -> Tensor:
        n, k = self._shape
        w = Tensor.empty((n, k), F32)
        check(_l().gq_int4_dequantize(context(), self._qt.storage.handle, self._scale.storage.handle,
                                      self._zero.storage.handle, n, k, self._group, w.storage.handle))
        return w

    def linear(self, input: Tensor, bias: Tensor | None = None, kernel: int = KERNEL_AUTO, out: Tensor | None = None) -> Tensor:
        n, k = self._shape
        out_shape, m = _check_linear("int4", input, bias, n, k)
        y = _output(out, out_shape)
        check(_l().gq_int4_linear(context(), input.storage.handle, input.offset, m, k, self._qt.storage.handle,
                                  self._scale.storage.handle, self._zero.storage.handle,
                                  bias.storage.handle if bias is not None else 0,
                                  bias.offset if bias is not None else 0, n, self._group, y.storage.handle, kernel))
        return y


    def linear_backward(self, grad: Tensor, need_input: bool = True, need_bias: bool = False):
        """(grad_input, grad_bias) of ``linear`` with the weight frozen (crates/grilly-infer/src/quant4.rs:447-480)."""
        n, k = self._shape
        m = _check_grad("int4", grad, n)
        gx = Tensor.empty(tuple(grad.shape[:-1]) + (k,), F32) if need_input else None
        gb = Tensor.empty((n,), F32) if need_bias else None
        check(_l().gq_int4_linear_backward(context(), grad.storage.handle, grad.offset, m, self._qt.storage.handle,
                                           self._scale.storage.handle, self._zero.storage.handle, n, k, self._group,
                                           gx.storage.handle if gx is not None else 0, gb.storage.handle if gb is not None else 0))
        return gx, gb


# ── capture, statistics (crates/grilly-py/src/ops.rs:484,584,611-657) ─────

class CommandGraph:
    """A recorded step. ``replay()`` re-runs it over the same buffers."""

    __slots__ = ("_g", "_nodes")

    def __init__(self, g, nodes) -> None:
        self._g, self._nodes = g, nodes

    def replay(self) -> None:
        check(_l().gq_graph_replay(context(), self._g))

    def __len__(self) -> int:
        return self._nodes

    def __repr__(self) -> str:
        return f"CommandGraph(commands={self._nodes})"

    def __del__(self) -> None:
        try:
            if self._g and _ctx is not None:
                _l().gq_graph_destroy(_ctx, self._g)
        except Exception:
            pass
        self._g = None


def begin_capture() -> None:
    check(_l().gq_begin_capture(context()))


def end_capture() -> CommandGraph:
    out = ctypes.c_void_p()
    check(_l().gq_end_capture(context(), ctypes.byref(out)))
    nodes = ctypes.c_uint64()
    check(_l().gq_graph_nodes(out, ctypes.byref(nodes)))
    return CommandGraph(out, nodes.value)


def abort_capture() -> None:
    """Close an open capture and discard it (an exception inside a captured step)."""
    _l().gq_end_capture(context(), None)


def capturing() -> bool:
    out = ctypes.c_uint32()
    check(_l().gq_capturing(context(), ctypes.byref(out)))
    return bool(out.value)


def synchronize() -> None:
    check(_l().gq_synchronize(context()))


def submit_stats() -> dict:
    s = _lib.Stats()
    check(_l().gq_stats_get(context(), ctypes.byref(s)))
    return {name: int(getattr(s, name)) for name, _ in _lib.Stats._fields_}


def reset_persistent_peak() -> None:
    check(_l().gq_persistent_peak_reset(context()))


def caps() -> dict:
    c = _lib.Caps()
    check(_l().gq_caps_get(context(), ctypes.byref(c)))
    return {"device_name": c.device_name.decode(), "cc": (c.cc_major, c.cc_minor), "sm_count": c.sm_count,
            "max_shared_per_block": c.max_shared_per_block, "total_memory": c.total_memory, "l2_bytes": c.l2_bytes}
