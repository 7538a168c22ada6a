"""ctypes front end to liboracle.so (oracle.c), with numpy in and out.

TEST INFRASTRUCTURE ONLY — a checker for the CUDA path, never a fallback.
Each wrapper names the reference shader its C function follows; the
arithmetic lives in oracle.c.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

__all__ = ["build", "words8", "words4", "quantize_q8", "dequantize_q8", "linear_q8", "linear_q8_tiled",
           "linear_q8_f64", "quantize_q4", "dequantize_q4", "linear_q4", "linear_q4_f64", "pack_levels_q4",
           "unpack_q8", "unpack_q4", "threads", "set_threads", "xorshift_data"]

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "liboracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile oracle.c with the Makefile beside it; returns the library path."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-s", "-B"], check=True)
    return _SO


def _load():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        i64, vp, ci = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int
        sig = {
            "oq_words8": ([i64], i64), "oq_words4": ([i64], i64),
            "oq_quantize_q8": ([vp, i64, i64, vp, vp], None),
            "oq_dequantize_q8": ([vp, vp, i64, i64, vp], None),
            "oq_linear_q8": ([vp, i64, i64, vp, vp, vp, i64, vp], None),
            "oq_linear_q8_tiled": ([vp, i64, i64, vp, vp, vp, i64, vp], None),
            "oq_linear_q8_f64": ([vp, i64, i64, vp, vp, vp, i64, vp, vp], None),
            "oq_quantize_q4": ([vp, i64, i64, i64, vp, vp, vp], None),
            "oq_dequantize_q4": ([vp, vp, vp, i64, i64, i64, vp], None),
            "oq_linear_q4": ([vp, i64, i64, vp, vp, vp, vp, i64, i64, ci, vp], None),
            "oq_linear_q4_f64": ([vp, i64, i64, vp, vp, vp, vp, i64, i64, vp, vp], None),
            "oq_pack_levels_q4": ([vp, i64, i64, vp], None),
            "oq_threads": ([], ci), "oq_set_threads": ([ci], None),
        }
        for name, (args, res) in sig.items():
            fn = getattr(_lib, name)
            fn.argtypes, fn.restype = args, res
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _f32(a, shape=None):
    a = np.ascontiguousarray(a, dtype=np.float32)
    if shape is not None:
        assert a.shape == tuple(shape), (a.shape, shape)
    return a


def words8(k: int) -> int:
    return -(-k // 16) * 4


def words4(k: int) -> int:
    return -(-k // 32) * 4


def threads() -> int:
    return _load().oq_threads()


def set_threads(n: int) -> None:
    _load().oq_set_threads(int(n))


def quantize_q8(w):
    """g2-quantize-q8.glsl -> (q uint32 (rows, words8), scale float32 (rows,))."""
    w = _f32(w)
    rows, k = w.shape
    q = np.empty((rows, words8(k)), dtype=np.uint32)
    scale = np.empty(rows, dtype=np.float32)
    _load().oq_quantize_q8(_p(w), rows, k, _p(q), _p(scale))
    return q, scale


def dequantize_q8(q, scale, k):
    q = np.ascontiguousarray(q, dtype=np.uint32)
    rows = q.shape[0]
    w = np.empty((rows, k), dtype=np.float32)
    _load().oq_dequantize_q8(_p(q), _p(_f32(scale, (rows,))), rows, k, _p(w))
    return w


def _lin8(fn, x, q, scale, bias, k):
    x = _f32(x)
    m = x.size // k if k else 0
    q = np.ascontiguousarray(q, dtype=np.uint32)
    n = q.shape[0]
    bias = None if bias is None else _f32(bias, (n,))
    y = np.empty((m, n), dtype=np.float32)
    fn(_p(x), m, k, _p(q), _p(_f32(scale, (n,))), _p(bias), n, _p(y))
    return y


def linear_q8(x, q, scale, bias, k):
    """g2-linear-q8.glsl (decode order), float32."""
    return _lin8(_load().oq_linear_q8, x, q, scale, bias, k)


def linear_q8_tiled(x, q, scale, bias, k):
    """g2-linear-q8-tiled.glsl (serial-k order), float32."""
    return _lin8(_load().oq_linear_q8_tiled, x, q, scale, bias, k)


def linear_q8_f64(x, q, scale, bias, k):
    """float64 value and the magnitude the reference's bound is stated in."""
    x = _f32(x)
    m = x.size // k
    q = np.ascontiguousarray(q, dtype=np.uint32)
    n = q.shape[0]
    bias = None if bias is None else _f32(bias, (n,))
    y, mag = np.empty((m, n)), np.empty((m, n))
    _load().oq_linear_q8_f64(_p(x), m, k, _p(q), _p(_f32(scale, (n,))), _p(bias), n, _p(y), _p(mag))
    return y, mag


def quantize_q4(w, group: int = 128):
    """g2-quantize-q4.glsl -> (q uint32 (rows, words4), scale, zero (rows, groups))."""
    w = _f32(w)
    rows, k = w.shape
    groups = -(-k // group)
    q = np.empty((rows, words4(k)), dtype=np.uint32)
    scale = np.empty((rows, groups), dtype=np.float32)
    zero = np.empty((rows, groups), dtype=np.float32)
    _load().oq_quantize_q4(_p(w), rows, k, group, _p(q), _p(scale), _p(zero))
    return q, scale, zero


def dequantize_q4(q, scale, zero, k, group: int = 128):
    q = np.ascontiguousarray(q, dtype=np.uint32)
    rows = q.shape[0]
    w = np.empty((rows, k), dtype=np.float32)
    _load().oq_dequantize_q4(_p(q), _p(_f32(scale)), _p(_f32(zero)), rows, k, group, _p(w))
    return w


def linear_q4(x, q, scale, zero, bias, k, group: int = 128, x_vec4=None):
    """g2-linear-q4.glsl, float32. x_vec4 defaults to the reference's rule for
    a tensor at offset 0: k % 4 == 0 (crates/grilly-infer/src/quant4.rs:423)."""
    x = _f32(x)
    m = x.size // k
    q = np.ascontiguousarray(q, dtype=np.uint32)
    n = q.shape[0]
    bias = None if bias is None else _f32(bias, (n,))
    if x_vec4 is None:
        x_vec4 = k % 4 == 0
    y = np.empty((m, n), dtype=np.float32)
    _load().oq_linear_q4(_p(x), m, k, _p(q), _p(_f32(scale)), _p(_f32(zero)), _p(bias), n, group, int(bool(x_vec4)),
                         _p(y))
    return y


def linear_q4_f64(x, q, scale, zero, bias, k, group: int = 128):
    x = _f32(x)
    m = x.size // k
    q = np.ascontiguousarray(q, dtype=np.uint32)
    n = q.shape[0]
    bias = None if bias is None else _f32(bias, (n,))
    y, mag = np.empty((m, n)), np.empty((m, n))
    _load().oq_linear_q4_f64(_p(x), m, k, _p(q), _p(_f32(scale)), _p(_f32(zero)), _p(bias), n, group, _p(y), _p(mag))
    return y, mag


def pack_levels_q4(levels):
    """Int4Tensor.from_parts' packer (python/grilly/infer/quantization.py:236-244)."""
    levels = np.ascontiguousarray(levels, dtype=np.uint8)
    rows, k = levels.shape
    q = np.empty((rows, words4(k)), dtype=np.uint32)
    _load().oq_pack_levels_q4(_p(levels), rows, k, _p(q))
    return q


def unpack_q8(q, k):
    """(rows, words8) words -> (rows, k) int8, padding stripped (Int8Weight::qdata)."""
    q = np.ascontiguousarray(q, dtype=np.uint32)
    return q.view(np.int8).reshape(q.shape[0], -1)[:, :k].copy()


def unpack_q4(q, k):
    """(rows, words4) words -> (rows, k) uint8 levels."""
    q = np.ascontiguousarray(q, dtype=np.uint32)
    b = q.view(np.uint8).reshape(q.shape[0], -1)
    out = np.empty((q.shape[0], b.shape[1] * 2), dtype=np.uint8)
    out[:, 0::2] = b & 0xF
    out[:, 1::2] = b >> 4
    return out[:, :k].copy()


def xorshift_data(n: int, seed: int, lo: float, hi: float, int4_form: bool = False):
    """The reference tests' seeded generator (crates/grilly-infer/tests/quant.rs:27-37;
    quant4.rs:28-39 multiplies in the other order, selected by int4_form)."""
    mask = (1 << 64) - 1
    s = ((seed * 0x9E3779B97F4A7C15) & mask) | 1
    out = np.empty(n, dtype=np.float32)
    lo32, hi32 = np.float32(lo), np.float32(hi)
    span = np.float32(hi32 - lo32)
    inv = np.float32(1 << 24)
    for i in range(n):
        s ^= (s << 13) & mask
        s ^= s >> 7
        s ^= (s << 17) & mask
        u = np.float32(np.float32(s >> 40) / inv)
        out[i] = lo32 + (u * span if int4_form else span * u)
    return out
