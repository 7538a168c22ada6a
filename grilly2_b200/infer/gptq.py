"""GPTQ with the heavy parts on the device — the counterpart of python/grilly/infer/gptq.py (numerics) and the
Hessian capture of python/grilly/infer/calibration.py:97-123.

    acc = HessianAccumulator(in_features)      # H = 2 X^T X, accumulated on the GPU as calibration rows arrive
    acc.add(x)                                  # x: (rows, in_features) float32 tensor
    w4 = gptq_quantize(weight, acc.hessian())  # an Int4Tensor, quantized column by column on the GPU

What stays on the host is what the reference also does there once per layer: damping H and factoring its inverse
(``_inverse_cholesky``, float64 numpy, K^3 work) — the column loop, N K^2 work and "most of" the reference's 263 s per
model (docs/inference.md:357-359), runs in CUDA (csrc/gptq.cu). ``act_order`` / ``static_groups`` are not implemented.
"""
from __future__ import annotations

import numpy as np

from .. import _C, _lib
from .._lib import check

__all__ = ["HessianAccumulator", "gptq_quantize", "inverse_cholesky"]


class HessianAccumulator:
    """H = 2 X^T X over every row of calibration input a layer sees, float32 on the device."""

    def __init__(self, in_features: int) -> None:
        self.k = int(in_features)
        self._h = _C.Tensor.from_numpy(np.zeros((self.k, self.k), dtype=np.float32), persistent=True)
        self.rows = 0

    def add(self, x) -> None:
        t = getattr(x, "_t", x)
        if t.dtype != "float32" or not t.shape or t.shape[-1] != self.k:
            raise RuntimeError(f"calibration rows must be float32 (..., {self.k}), got {t.dtype} {list(t.shape)}")
        rows = t.numel() // self.k
        check(_lib.load().gq_gptq_hessian_add(_C.context(), t.storage.handle, t.offset, rows, self.k, self._h.storage.handle))
        self.rows += rows

    def hessian(self) -> np.ndarray:
        return self._h.numpy()


def inverse_cholesky(hessian: np.ndarray, percdamp: float = 0.01):
    """The upper triangular U with U^T U = H^-1, damped as GPTQ does (gptq.py:68-84), in float64; and which input
    features were never excited (their weights are zeroed and their diagonal set to one)."""
    h = np.array(hessian, dtype=np.float64, copy=True)
    dead = np.diag(h) == 0.0
    h[dead, dead] = 1.0
    h[np.diag_indices_from(h)] += percdamp * np.mean(np.diag(h))
    lower_inv = np.linalg.inv(np.linalg.cholesky(h))
    return np.linalg.cholesky(lower_inv.T @ lower_inv).T, dead


def gptq_quantize(weight, hessian: np.ndarray, group_size: int = 128, percdamp: float = 0.01, act_order: bool = False,
                  static_groups: bool | None = None):
    """``weight``: (out, in) float32 tensor (or numpy array); ``hessian``: (in, in). Returns an ``Int4Tensor``."""
    from .quantization import Int4Tensor
    if act_order or static_groups:
        raise NotImplementedError("grilly: gptq_quantize with act_order / static_groups is not implemented yet")
    t = getattr(weight, "_t", weight)
    if isinstance(t, np.ndarray):
        t = _C.Tensor.from_numpy(np.ascontiguousarray(t, dtype=np.float32))
    if t.dtype != "float32" or len(t.shape) != 2:
        raise RuntimeError(f"expected a 2-D float32 weight (out_features, in_features), got {t.dtype} {list(t.shape)}")
    n, k = t.shape
    hessian = np.asarray(hessian)
    if hessian.shape != (k, k):
        raise ValueError(f"hessian must be ({k}, {k}) for a weight with {k} input features, got {tuple(hessian.shape)}")
    if group_size <= 0 or k % group_size:
        raise ValueError(f"in_features {k} must be a whole number of groups of {group_size}")
    upper, dead = inverse_cholesky(hessian, percdamp)
    work = t.clone_data()  # the loop consumes its working copy
    if dead.any():
        host = work.numpy()
        host[:, dead] = 0.0
        work = _C.Tensor.from_numpy(host)
    groups, words = k // group_size, -(-k // 32) * 4
    q = _C.Tensor.empty((n, words), "int32", persistent=True)
    scale = _C.Tensor.empty((n, groups), "float32", persistent=True)
    zero = _C.Tensor.empty((n, groups), "float32", persistent=True)
    u = _C.Tensor.from_numpy(upper.astype(np.float32))
    errors = _C.Tensor.empty((n, 128), "float32")
    check(_lib.load().gq_gptq_quantize(_C.context(), work.storage.handle, n, k, group_size, u.storage.handle, errors.storage.handle,
                                       q.storage.handle, scale.storage.handle, zero.storage.handle))
    return Int4Tensor._holding(_C.Int4Weight(q, scale, zero, (n, k), group_size))
