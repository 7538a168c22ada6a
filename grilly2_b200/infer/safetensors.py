"""Streaming safetensors reader: one tensor on the device at a time
(python/grilly/infer/safetensors.py:85-127; crates/grilly-infer/src/safetensors.rs:85-167).

The file is memory-mapped and its JSON header parsed here; tensors are widened
to what the device holds — F32 and I32 as they are, BF16 by a 16-bit shift,
F16 exactly, I64 narrowed to int32 when it fits, BOOL to 0/1 — and uploaded
one by one in file order.
"""
from __future__ import annotations

import json
import mmap
import struct

import numpy as np

from .. import Tensor, from_numpy

__all__ = ["safe_open", "stream_into", "load_file"]


def _widen(raw: np.ndarray, dtype: str, shape) -> np.ndarray:
    if dtype == "F32":
        return raw.view(np.float32).reshape(shape)
    if dtype == "BF16":
        return (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32).reshape(shape)
    if dtype == "F16":
        return raw.view(np.float16).astype(np.float32).reshape(shape)
    if dtype == "I32":
        return raw.view(np.int32).reshape(shape)
    if dtype == "I64":
        wide = raw.view(np.int64).reshape(shape)
        if wide.size and (wide.max() > np.iinfo(np.int32).max or wide.min() < np.iinfo(np.int32).min):
            raise NotImplementedError("grilly: int64 values beyond int32 are not implemented yet")
        return wide.astype(np.int32)
    if dtype == "BOOL":
        return raw.view(np.uint8).astype(np.int32).reshape(shape)
    raise NotImplementedError(f"grilly: safetensors dtype {dtype} is not implemented yet")


class safe_open:
    """``with safe_open(path) as f: f.keys(); f.get_tensor(name)``."""

    def __init__(self, filename, framework: str = "pt", device=None) -> None:
        self._file = open(filename, "rb")
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        if len(self._map) < 8:
            raise RuntimeError(f"{filename}: not a safetensors file (shorter than its length prefix)")
        (n,) = struct.unpack("<Q", self._map[:8])
        if 8 + n > len(self._map):
            raise RuntimeError(f"{filename}: header length {n} exceeds the file")
        header = json.loads(self._map[8:8 + n].decode("utf-8"))
        self._meta = header.pop("__metadata__", None)
        self._base = 8 + n
        self._entries = header
        for name, e in header.items():
            lo, hi = e["data_offsets"]
            if lo > hi or self._base + hi > len(self._map):
                raise RuntimeError(f"{filename}: tensor {name} lies outside the file")

    def __enter__(self):
        return self

    def __exit__(self, *exc) -> bool:
        self._map.close()
        self._file.close()
        return False

    def keys(self) -> list[str]:
        return sorted(self._entries)

    def offset_keys(self) -> list[str]:
        """Names in file order, which is the order a streaming load reads them in."""
        return sorted(self._entries, key=lambda k: self._entries[k]["data_offsets"][0])

    def metadata(self):
        return self._meta

    def get_slice_shape(self, name: str):
        return tuple(self._entries[name]["shape"])

    def get_tensor(self, name: str) -> Tensor:
        if name not in self._entries:
            raise KeyError(name)
        e = self._entries[name]
        lo, hi = e["data_offsets"]
        raw = np.frombuffer(self._map, dtype=np.uint8, count=hi - lo, offset=self._base + lo)
        return from_numpy(_widen(raw, e["dtype"], tuple(e["shape"])), persistent=True)  # weights: exact-size, counted


def load_file(filename, device="cpu") -> dict:
    with safe_open(filename) as f:
        return {k: f.get_tensor(k) for k in f.offset_keys()}


def stream_into(model, filename, strict: bool = True, convert=None) -> set[str]:
    """Load ``filename`` into ``model`` tensor by tensor; ``convert(key,
    tensor)`` may return a replacement (a quantized weight) or None to assign
    the tensor itself. Nothing keeps a tensor after its key is done."""
    own = {k: tuple(v.shape) for k, v in model.state_dict(keep_vars=True).items()}
    unexpected, errors = [], []
    with safe_open(filename) as f:
        names = f.offset_keys()
        for key in names:
            shape = own.get(key)
            if shape is None:
                unexpected.append(key)
                continue
            if f.get_slice_shape(key) != shape:
                errors.append(f"size mismatch for {key}: copying a param with shape {list(f.get_slice_shape(key))} "
                              f"from checkpoint, the shape in current model is {list(shape)}.")
                continue
            value = f.get_tensor(key)
            replacement = None if convert is None else convert(key, value)
            owner, _, attr = key.rpartition(".")
            target = model.get_submodule(owner)
            if replacement is None:
                model.load_state_dict({key: value}, assign=True, strict=False)
            else:
                setattr(target, attr, replacement)
            del value, replacement
    if strict:
        missing = [k for k in own if k not in set(names)]
        if missing:
            errors.insert(0, "Missing key(s) in state_dict: " + ", ".join(f'"{k}"' for k in missing))
        if unexpected:
            errors.insert(0, "Unexpected key(s) in state_dict: " + ", ".join(f'"{k}"' for k in unexpected))
    if errors:
        raise RuntimeError(f"Error(s) in loading state_dict for {type(model).__name__}:\n\t" + "\n\t".join(errors))
    return set(names)
