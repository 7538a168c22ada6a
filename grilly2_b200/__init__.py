"""grilly2_b200 — a B200 (sm_100a) backend for grilly2's weight-only quantized
linear path, behind grilly2's own Python surface for that path:

    from grilly2_b200.infer.quantization import quantize_, Int8WeightOnlyConfig
    quantize_(model, Int8WeightOnlyConfig())

Only what the path needs is here: a tensor handle (``from_numpy`` /
``.numpy()``), ``nn.Linear`` with the ``F.linear`` hook quantized weights use,
the quantization API, the streaming safetensors loader and ``graphed``.
Everything runs in hand-written CUDA kernels reached through the C ABI of
include/gq.h; there is no CPU path, and a missing library or GPU raises.
"""
from __future__ import annotations

import builtins as _builtins

import numpy as _np

from . import _C

__all__ = ["Size", "Tensor", "device", "empty", "float32", "from_numpy", "graphed", "int32", "no_grad", "tensor",
           "zeros", "synchronize"]


def _not_yet(what: str) -> NotImplementedError:
    return NotImplementedError(f"grilly: {what} is not implemented yet")


class dtype:
    __slots__ = ("name",)

    def __init__(self, name: str) -> None:
        self.name = name

    def __repr__(self) -> str:
        return f"grilly.{self.name}"


float32 = dtype("float32")
int32 = dtype("int32")
_DTYPES = {"float32": float32, "int32": int32}


class Size(tuple):
    def numel(self) -> int:
        return int(_np.prod(self, dtype=_np.int64)) if self else 1

    def __repr__(self) -> str:
        return f"grilly.Size({list(self)})"


class device:
    """Like ``torch.device``. The reference reports its one device as
    ``device(type='vulkan', index=0)`` and accepts ``"cpu"`` as an alias
    (python/grilly/__init__.py:123-191); a drop-in keeps that surface, although
    the memory behind it here is a B200's."""

    __slots__ = ("type", "index")

    def __init__(self, type, index=None) -> None:  # noqa: A002
        if isinstance(type, device):
            self.type, self.index = type.type, type.index
            return
        if isinstance(type, _builtins.int):
            type, index = "cuda", type
        if ":" in type:
            type, _, idx = type.partition(":")
            index = _builtins.int(idx)
        self.type, self.index = type, index

    def __eq__(self, other) -> bool:
        return isinstance(other, device) and (self.type, self.index) == (other.type, other.index)

    def __hash__(self) -> int:
        return hash((self.type, self.index))

    def __str__(self) -> str:
        return self.type if self.index is None else f"{self.type}:{self.index}"

    def __repr__(self) -> str:
        return f"device(type='{self.type}'" + ("" if self.index is None else f", index={self.index}") + ")"


_DEVICE = device("vulkan", 0)


def _resolve_device(d) -> device:
    if d is None:
        return _DEVICE
    dev = device(d)
    if dev.type in ("vulkan", "cpu") and dev.index in (None, 0):
        return _DEVICE
    raise _not_yet(f"device {str(dev)!r} (grilly runs on one device; 'cpu' is accepted as an alias for it)")


class Tensor:
    """A device tensor. ``_t`` is the core handle the compiled side works on
    (python/grilly/__init__.py:273-287)."""

    __slots__ = ("_core", "_grad", "__weakref__")

    def __init__(self, *args, **kwargs) -> None:
        raise _not_yet("the legacy Tensor(...) constructor; use tensor(...) or from_numpy(...)")

    @classmethod
    def _wrap(cls, core: _C.Tensor) -> "Tensor":
        t = object.__new__(cls)
        t._core, t._grad = core, None
        return t

    @property
    def _t(self) -> _C.Tensor:
        return self._core

    @property
    def shape(self) -> Size:
        return Size(self._t.shape)

    def size(self, dim=None):
        return self.shape if dim is None else self.shape[dim]

    def dim(self) -> int:
        return len(self.shape)

    def numel(self) -> int:
        return self.shape.numel()

    @property
    def dtype(self):
        return _DTYPES[self._t.dtype]

    @property
    def device(self) -> device:
        return _DEVICE

    @property
    def requires_grad(self) -> bool:
        return False

    def requires_grad_(self, requires_grad: bool = True) -> "Tensor":
        if requires_grad:
            raise _not_yet("autograd (this backend is the inference path: weights are frozen and steps run under no_grad)")
        return self

    @property
    def grad(self):
        return None

    def detach(self) -> "Tensor":
        return self

    def numpy(self) -> _np.ndarray:
        """A host copy; waits for the device."""
        return self._t.numpy()

    def tolist(self):
        return self.numpy().tolist()

    def clone(self) -> "Tensor":
        return Tensor._wrap(self._t.clone_data())

    def copy_(self, src: "Tensor") -> "Tensor":
        self._t.copy_(_require_tensor("src", src)._t)
        return self

    def reshape(self, *shape) -> "Tensor":
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        n = self.numel()
        if -1 in shape:
            known = -int(_np.prod(shape, dtype=_np.int64))
            shape = tuple(n // known if s == -1 else s for s in shape)
        return Tensor._wrap(self._t.reshape(shape))

    view = reshape

    def __len__(self) -> int:
        return self.shape[0]

    def __repr__(self) -> str:
        return f"tensor({_np.array2string(self.numpy(), separator=', ')}, device='{_DEVICE}')"


def _require_tensor(name: str, value) -> Tensor:
    if not isinstance(value, Tensor):
        raise TypeError(f"{name} must be a Tensor, got {type(value).__name__}")
    return value


def from_numpy(array, persistent: bool = False) -> Tensor:
    """A device tensor holding a copy of ``array`` (float32 or int32).
    ``persistent`` places it in exact-size, counted memory, where weights live."""
    return Tensor._wrap(_C.Tensor.from_numpy(_np.asarray(array), persistent))


def tensor(data, dtype=None, device=None, requires_grad: bool = False) -> Tensor:
    _resolve_device(device)
    a = _np.asarray(data)
    if dtype is None:
        a = a.astype(_np.float32) if a.dtype.kind == "f" else a.astype(_np.int32) if a.dtype.kind in "iu" else a
    else:
        a = a.astype(_np.float32 if dtype is float32 else _np.int32)
    t = from_numpy(a)
    return t.requires_grad_(requires_grad) if requires_grad else t


def zeros(*shape, dtype=None, device=None) -> Tensor:
    if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
        shape = tuple(shape[0])
    return tensor(_np.zeros(shape, dtype=_np.float32), dtype=dtype, device=device)


def empty(*shape, dtype=None, device=None) -> Tensor:
    if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
        shape = tuple(shape[0])
    _resolve_device(device)
    return Tensor._wrap(_C.Tensor.empty(shape, "int32" if dtype is int32 else "float32"))


class no_grad:
    """Accepted for source compatibility: nothing here records gradients."""

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False

    def __call__(self, fn):
        return fn


def synchronize() -> None:
    _C.synchronize()


from ._graph import graphed  # noqa: E402
from . import nn  # noqa: E402,F401
