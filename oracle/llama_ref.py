"""float64 numpy model of one decode step of the int8 weight-only Llama/Qwen2
decoder. TEST INFRASTRUCTURE ONLY (a checker for grilly2_b200.infer.llama).

It follows the reference's own float64 model of its fused step,
``reference_logits`` in tests/python/test_fused_ops.py:135-171, with the int8
weights taken as the oracle quantizes them (oracle.quantize_q8, pinned
against the reference's formula) and every product in float64:
  h = embed[token]
  per layer: x = rms_norm(h) w;  q,k,v = x Wqkv^T + b;  rotary(q, k) at the cache length;
             append k, v;  a = softmax(q K^T / sqrt(d)) V per head (grouped);  h += a Wo^T;
             x = rms_norm(h) w;  h += (silu(x Wg^T) * (x Wu^T)) Wd^T
  logits = rms_norm(h) w  Wembed_q^T
"""
from __future__ import annotations

import numpy as np

from . import oracle


def _deq(w: np.ndarray) -> np.ndarray:
    q, s = oracle.quantize_q8(w)
    return oracle.dequantize_q8(q, s, w.shape[1]).astype(np.float64)


class DecoderRef:
    def __init__(self, cfg, weights: dict, cos: np.ndarray, sin: np.ndarray, int8_kv: bool = False) -> None:
        self.cfg = cfg
        self.int8_kv = int8_kv  # cached rows stored as rint(v / s) * s, s = float32(max|v|) / 127, as the int8 cache does
        self.embed = weights["embed"].astype(np.float64)
        self.head = _deq(weights["embed"])
        self.norm = weights["norm"].astype(np.float64)
        self.cos, self.sin = cos.astype(np.float64), sin.astype(np.float64)
        self.layers = []
        for lw in weights["layers"]:
            self.layers.append({k: (_deq(v) if v.ndim == 2 else v.astype(np.float64)) for k, v in lw.items()})
        c = cfg
        self.k = np.zeros((c.num_hidden_layers, c.num_key_value_heads, c.max_cache_len, c.head_dim))
        self.v = np.zeros_like(self.k)
        self.length = 0

    def fill(self, k, v, length):
        self.k[:, :, :length], self.v[:, :, :length], self.length = k, v, length

    def _rms(self, h, w):
        return h / np.sqrt(np.mean(h * h) + self.cfg.rms_norm_eps) * w

    def _rope(self, x, pos):
        d = self.cfg.head_dim
        x = x.reshape(-1, d)
        rot = np.concatenate([-x[:, d // 2:], x[:, :d // 2]], axis=1)
        return x * self.cos[pos] + rot * self.sin[pos]

    def _stored(self, rows):
        """What the cache holds for these rows: themselves, or their int8 codes times the row's scale (the rows reach
        the cache as float32, so the scale and the codes are formed from the float32 values)."""
        if not self.int8_kv:
            return rows
        r32 = rows.astype(np.float32)
        amax = np.abs(r32).max(axis=-1, keepdims=True)
        scale = np.where(amax > 0, (amax / np.float32(127.0)).astype(np.float32), np.float32(1.0)).astype(np.float32)
        codes = np.clip(np.rint((r32 / scale).astype(np.float32)), -127, 127)
        return codes.astype(np.float64) * scale.astype(np.float64)

    def step(self, token: int) -> np.ndarray:
        c = self.cfg
        pos = self.length
        h = self.embed[token].copy()
        for li, lw in enumerate(self.layers):
            x = self._rms(h, lw["input_norm"])
            q = lw["q"] @ x + lw["q_bias"]
            k = lw["k"] @ x + lw["k_bias"]
            v = lw["v"] @ x + lw["v_bias"]
            q, k = self._rope(q, pos), self._rope(k, pos)
            if pos < c.max_cache_len:
                self.k[li, :, pos], self.v[li, :, pos] = self._stored(k), self._stored(v.reshape(-1, c.head_dim))
            n = min(pos + 1, c.max_cache_len)
            out = np.zeros((c.num_attention_heads, c.head_dim))
            rep = c.num_attention_heads // c.num_key_value_heads
            for hh in range(c.num_attention_heads):
                g = hh // rep
                s = self.k[li, g, :n] @ q[hh] / np.sqrt(c.head_dim)
                e = np.exp(s - s.max())
                out[hh] = (e / e.sum()) @ self.v[li, g, :n]
            h = h + lw["o"] @ out.reshape(-1)
            x = self._rms(h, lw["post_norm"])
            g_, u_ = lw["gate"] @ x, lw["up"] @ x
            h = h + lw["down"] @ (g_ / (1.0 + np.exp(-g_)) * u_)
        self.length = min(pos + 1, c.max_cache_len)
        return self.head @ self._rms(h, self.norm)
