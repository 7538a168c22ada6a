"""Weight-only int8 / int4 quantization with torchao's surface, as the
reference exposes it (python/grilly/infer/quantization.py):

    quantize_(model, Int8WeightOnlyConfig())        # per output row, symmetric
    quantize_(model, Int4WeightOnlyConfig())        # groups of 128, asymmetric
    load_quantized_(model, "model.safetensors", Int8WeightOnlyConfig())

Numerics (bit-exact with the reference; see csrc/quantize.cu):
  int8   scale = max|w| / 127.5 per row (>= float32 eps);
         q = clamp(round_half_even(w * (1 / scale)), -128, 127)
  int4   per group: scale = (max - min) / 15 (>= eps); zero = min + 8 * scale;
         level = clamp(round_half_even((w - min) / scale), 0, 15);
         dequantize = level * scale + (zero - 8 * scale)

A quantized weight is frozen, lives in persistent device memory, and runs
``F.linear`` through its own dequant-fused kernel; every other use of it sees
the dequantized float32 weight, computed on demand.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from .. import Size, Tensor, _C, _DEVICE, _not_yet, _require_tensor, _resolve_device, float32, from_numpy
from ..nn.modules import Linear, Parameter

__all__ = ["Int4Tensor", "Int4WeightOnlyConfig", "Int8Tensor", "Int8WeightOnlyConfig", "PerRow", "QuantizedTensor",
           "load_packed_", "load_quantized_", "quantize_", "save_packed"]


@dataclass(frozen=True)
class PerRow:
    """torchao.quantization.PerRow: one scale per output feature."""

    dim: int = -1


def _refuse_version_1(config_name: str, version: int) -> None:
    if version == 1:
        raise ValueError(f"version 1 of {config_name} has been removed, please use version 2")


@dataclass
class Int8WeightOnlyConfig:
    """torchao's ``Int8WeightOnlyConfig`` (version 2), per-row only."""

    group_size: int | None = None
    granularity: object = field(default_factory=PerRow)
    set_inductor_config: bool = True
    version: int = 2

    def __post_init__(self) -> None:
        _refuse_version_1("Int8WeightOnlyConfig", self.version)
        assert self.group_size is None, (f"Only support version 2 with group_size=None, got {self.group_size}. "
                                         f"Use granularity=PerGroup({self.group_size}) instead.")
        if self.granularity != PerRow():
            raise _not_yet(f"Int8WeightOnlyConfig(granularity={self.granularity!r}) (grilly has PerRow())")


@dataclass
class Int4WeightOnlyConfig:
    """torchao's ``Int4WeightOnlyConfig``: ``group_size`` values share a scale
    and a zero point. A 16-byte vector holds 32 levels and must lie inside one
    group, hence the multiple of 32."""

    group_size: int = 128
    version: int = 2

    def __post_init__(self) -> None:
        _refuse_version_1("Int4WeightOnlyConfig", self.version)
        g = self.group_size
        if not isinstance(g, int) or g <= 0 or g % 32:
            raise ValueError(f"group_size must be a positive multiple of 32, got {g}")


class QuantizedTensor(Parameter):
    """Common part of the quantized weights: the float weight's shape and
    dtype, no gradient, and ``_q`` holding the packed device data."""

    __slots__ = ("_q",)

    def __new__(cls, *args, **kwargs):
        raise TypeError(f"create a {cls.__name__} with {cls.__name__}.from_hp(weight)")

    def __init__(self, *args, **kwargs) -> None:
        pass

    @classmethod
    def _holding(cls, q):
        t = object.__new__(cls)
        t._q, t._grad = q, None
        return t

    @property
    def _t(self):  # anything but F.linear works on the dequantized weight
        return self._q.dequantize()

    def dequantize(self, output_dtype=None) -> Tensor:
        if output_dtype not in (None, float32):
            raise _not_yet(f"dequantize(output_dtype={output_dtype!r})")
        return Tensor._wrap(self._q.dequantize())

    @property
    def nbytes(self) -> int:
        """Device bytes of the packed values and their parameters."""
        return self._q.nbytes

    def _grilly_linear(self, input, bias):
        x = _require_tensor("input", input)
        b = None if bias is None else _require_tensor("bias", bias)._t
        return Tensor._wrap(self._q.linear(x._t, b))

    @property
    def shape(self) -> Size:
        return Size(self._q.shape)

    def dim(self) -> int:
        return 2

    def numel(self) -> int:
        n, k = self._q.shape
        return n * k

    @property
    def dtype(self):
        return float32

    @property
    def device(self):
        return _DEVICE

    @property
    def requires_grad(self) -> bool:
        return False

    @requires_grad.setter
    def requires_grad(self, value) -> None:
        self.requires_grad_(value)

    def requires_grad_(self, requires_grad: bool = True):
        if requires_grad:
            raise RuntimeError(f"an {type(self).__name__} weight is frozen: gradients reach the layer's input and bias only")
        return self

    is_leaf = True
    grad_fn = None

    @property
    def grad(self):
        return None

    @grad.setter
    def grad(self, value) -> None:
        if value is not None:
            raise RuntimeError(f"an {type(self).__name__} weight has no gradient")


class Int8Tensor(QuantizedTensor):
    """int8 values with one float32 scale per output row (torchao's ``Int8Tensor``)."""

    __slots__ = ()

    @classmethod
    def from_hp(cls, hp_tensor, granularity=None) -> "Int8Tensor":
        if granularity is not None and granularity != PerRow():
            raise _not_yet(f"Int8Tensor.from_hp(granularity={granularity!r}) (grilly has PerRow())")
        return cls._holding(_C.Int8Weight.quantize(_require_tensor("hp_tensor", hp_tensor)._t))

    @classmethod
    def _cat(cls, parts) -> "Int8Tensor":
        """The parts' rows as one weight (a fused q/k/v or gate/up projection);
        exact, because scales are per row."""
        return cls._holding(_C.Int8Weight.cat([p._q for p in parts]))

    @property
    def scale(self) -> Tensor:
        return Tensor._wrap(self._q.scale())

    def __repr__(self) -> str:
        n, k = self._q.shape
        return f"Int8Tensor(shape=({n}, {k}), granularity=PerRow(), nbytes={self.nbytes})"


class Int4Tensor(QuantizedTensor):
    """4-bit levels with a float32 scale and zero point per group (torchao's ``Int4Tensor``)."""

    __slots__ = ()

    @classmethod
    def from_hp(cls, hp_tensor, group_size: int = 128) -> "Int4Tensor":
        return cls._holding(_C.Int4Weight.quantize(_require_tensor("hp_tensor", hp_tensor)._t, int(group_size)))

    @classmethod
    def from_parts(cls, levels, scales, zeros, group_size: int = 128) -> "Int4Tensor":
        """Install levels (out, in) of 0..15 and per-group parameters (out,
        groups) chosen elsewhere — by GPTQ, say. Packing: eight levels per
        32-bit word, low nibble first, rows padded to whole 16-byte vectors."""
        levels = np.ascontiguousarray(levels, dtype=np.uint8)
        n, k = levels.shape
        words = -(-k // 32) * 4
        padded = np.zeros((n, words * 8), dtype=np.uint32)
        padded[:, :k] = levels
        shifts = (4 * np.arange(8, dtype=np.uint32))[None, None, :]
        packed = np.bitwise_or.reduce(padded.reshape(n, words, 8) << shifts, axis=2).astype(np.uint32)
        return cls._holding(_C.Int4Weight.from_parts(
            from_numpy(packed.view(np.int32))._t, from_numpy(np.ascontiguousarray(scales, dtype=np.float32))._t,
            from_numpy(np.ascontiguousarray(zeros, dtype=np.float32))._t, k, int(group_size)))

    @classmethod
    def _cat(cls, parts) -> "Int4Tensor":
        return cls._holding(_C.Int4Weight.cat([p._q for p in parts]))

    @property
    def group_size(self) -> int:
        return self._q.group_size

    @property
    def scale(self) -> Tensor:
        return Tensor._wrap(self._q.scale())

    @property
    def zero(self) -> Tensor:
        return Tensor._wrap(self._q.zero())

    def __repr__(self) -> str:
        n, k = self._q.shape
        return f"Int4Tensor(shape=({n}, {k}), group_size={self.group_size}, nbytes={self.nbytes})"


def _is_linear(mod, *args) -> bool:
    """torchao's default filter: an ``nn.Linear`` whose weight is still float."""
    return isinstance(mod, Linear) and hasattr(mod, "weight") and not isinstance(mod.weight, QuantizedTensor)


_SUPPORTED = "(grilly has Int8WeightOnlyConfig and Int4WeightOnlyConfig)"


def _quantized(weight, config):
    if isinstance(config, Int8WeightOnlyConfig):
        return Int8Tensor.from_hp(weight, config.granularity)
    if isinstance(config, Int4WeightOnlyConfig):
        return Int4Tensor.from_hp(weight, config.group_size)
    raise _not_yet(f"quantizing with {type(config).__name__} {_SUPPORTED}")


def quantize_(model, config, filter_fn=_is_linear, device=None) -> None:
    """Replace, in place, the weight of every module of ``model`` (itself
    included) for which ``filter_fn(module, qualified_name)`` holds."""
    if not isinstance(config, (Int8WeightOnlyConfig, Int4WeightOnlyConfig)):
        raise _not_yet(f"quantize_ with {type(config).__name__} {_SUPPORTED}")
    if device is not None:
        _resolve_device(device)
    for name, module in list(model.named_modules()):
        if filter_fn(module, name):
            module.weight = _quantized(module.weight, config)


def load_quantized_(model, filename, config, filter_fn=_is_linear, strict: bool = True) -> set[str]:
    """Stream a safetensors checkpoint into ``model``, quantizing each selected
    weight as it arrives, so that one float32 tensor is alive at a time
    instead of all of them beside their quantized copies. The result is the
    same tensors, bit for bit, as load-then-``quantize_``. Returns the names
    the file held; ``strict`` reports missing and unexpected names as
    ``load_state_dict`` does."""
    from .safetensors import stream_into

    wanted = {(f"{name}.weight" if name else "weight") for name, module in model.named_modules()
              if filter_fn(module, name)}

    def convert(key, value):
        return _quantized(value, config) if key in wanted else None

    return stream_into(model, filename, strict=strict, convert=convert)


# ── pre-packed checkpoints ────────────────────────────────────────────────
# The reference quantizes at load time from a float checkpoint (load_quantized_ above) and names a checkpoint that
# already holds the packed weights as its next step (docs/inference.md:900-904). This is that step: a safetensors file
# whose quantized weights are stored as they lie on the device — `<name>.__q` (int32 words), `<name>.__scale` and, for
# int4, `<name>.__zero` — with the packing described in the metadata. Loading uploads each packed tensor straight into
# persistent device memory: no float32 copy of a quantized weight exists at any point, on the host or the device.

_PACKED = "grilly_packed"


def save_packed(model, filename) -> set[str]:
    """Write ``model``'s parameters to ``filename`` (safetensors): quantized weights packed, the rest float32 / int32 as
    they are. Returns the tensor names written."""
    import json
    import struct

    import numpy as np
    entries, blobs, meta, at = {}, [], {_PACKED: "1"}, 0

    def add(name, arr):
        nonlocal at
        arr = np.ascontiguousarray(arr)
        dtype = {"float32": "F32", "int32": "I32"}[str(arr.dtype)]
        entries[name] = {"dtype": dtype, "shape": list(arr.shape), "data_offsets": [at, at + arr.nbytes]}
        blobs.append(arr.tobytes())
        at += arr.nbytes

    for name, p in model.state_dict(keep_vars=True).items():
        if isinstance(p, Int8Tensor):
            add(name + ".__q", p._q.packed().numpy())
            add(name + ".__scale", p._q.scale().numpy())
            meta[name] = json.dumps({"bits": 8, "shape": list(p.shape)})
        elif isinstance(p, Int4Tensor):
            add(name + ".__q", p._q.packed().numpy())
            add(name + ".__scale", p._q.scale().numpy())
            add(name + ".__zero", p._q.zero().numpy())
            meta[name] = json.dumps({"bits": 4, "shape": list(p.shape), "group_size": p.group_size})
        else:
            add(name, p.numpy())
    header = json.dumps({"__metadata__": meta, **entries}, separators=(",", ":")).encode("utf-8")
    header += b" " * (-len(header) % 8)
    with open(filename, "wb") as f:
        f.write(struct.pack("<Q", len(header)))
        f.write(header)
        for b in blobs:
            f.write(b)
    return set(entries)


def load_packed_(model, filename, strict: bool = True) -> set[str]:
    """Load a ``save_packed`` file into ``model``, tensor by tensor. A packed weight replaces the module's float weight
    with the quantized tensor the file describes (whatever the module held before); nothing is quantized or dequantized.
    Returns the parameter names the file held."""
    import json

    from .. import _C
    from .safetensors import safe_open
    own = set(model.state_dict(keep_vars=True))
    seen: set[str] = set()
    with safe_open(filename) as f:
        meta = f.metadata() or {}
        if meta.get(_PACKED) != "1":
            raise RuntimeError(f"{filename} is not a pre-packed checkpoint (no {_PACKED} marker): load it with load_quantized_")
        packed = {k: json.loads(v) for k, v in meta.items() if k != _PACKED}
        names = f.offset_keys()
        plain = [k for k in names if ".__" not in k]
        unexpected = [k for k in list(packed) + plain if k not in own]
        if strict and unexpected:
            raise RuntimeError("Unexpected key(s) in state_dict: " + ", ".join(f'"{k}"' for k in unexpected))
        for key in plain:
            if key in own:
                model.load_state_dict({key: f.get_tensor(key)}, assign=True, strict=False)
                seen.add(key)
        for key, info in packed.items():
            if key not in own:
                continue
            n, k = info["shape"]
            q = f.get_tensor(key + ".__q")._t        # int32 words, uploaded as they are into persistent memory
            scale = f.get_tensor(key + ".__scale")._t
            if info["bits"] == 8:
                if tuple(q.shape) != (n, -(-k // 16) * 4) or tuple(scale.shape) != (n,):
                    raise RuntimeError(f"{key}: packed int8 tensors {list(q.shape)} / {list(scale.shape)} do not describe a ({n}, {k}) weight")
                value = Int8Tensor._holding(_C.Int8Weight(q, scale, (n, k)))
            else:
                zero = f.get_tensor(key + ".__zero")._t
                value = Int4Tensor._holding(_C.Int4Weight.from_parts(q, scale, zero, k, int(info["group_size"])))
            owner, _, attr = key.rpartition(".")
            setattr(model.get_submodule(owner), attr, value)
            seen.add(key)
            del q, scale, value
    if strict:
        missing = [k for k in own if k not in seen]
        if missing:
            raise RuntimeError("Missing key(s) in state_dict: " + ", ".join(f'"{k}"' for k in missing))
    return seen
