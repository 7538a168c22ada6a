"""One decode step of a Llama/Qwen2-shaped causal LM with int8 weight-only
linears — the no-grad fused path of the reference's ``LlamaForCausalLM``
(python/grilly/infer/models/llama.py:340-366): embedding, then per layer
add+RMSNorm -> fused q|k|v int8 linear (+bias) -> rotary into the KV cache ->
grouped-query decode attention -> o_proj int8 -> add+RMSNorm -> fused gate|up
int8 -> SwiGLU -> down int8; final norm; tied lm_head int8 (the embedding table
itself stays float32). Fused weights are the rows of the parts stacked
(``Int8Weight.cat``, exact because scales are per row).

Unlike the reference's step, nothing here depends on a host integer: the token
id, the cache cursor and with it q's rotary position are read on the device, so
``grilly2_b200.graphed(model.step)`` replays correctly from the second call on.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import numpy as np

from .. import _C, _lib
from .._lib import check


@dataclass
class LlamaConfig:
    vocab_size: int = 151936
    hidden_size: int = 896
    num_hidden_layers: int = 24
    num_attention_heads: int = 14
    num_key_value_heads: int = 2
    head_dim: int = 64
    intermediate_size: int = 4864
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    max_cache_len: int = 1024
    attention_bias: bool = True  # Qwen2: q, k, v carry a bias (python/grilly/huggingface/configuration.py:134)

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim


def qwen25_05b(max_cache_len: int = 1024) -> LlamaConfig:
    """The Qwen2.5-0.5B architecture (weights are random-initialised by the caller)."""
    return LlamaConfig(max_cache_len=max_cache_len)


def rotary_tables(cfg: LlamaConfig):
    """cos / sin [max_cache_len, head_dim] in float32, as transformers builds them:
    inv_freq = theta^(-2i/d), angles = position * inv_freq, emb = cat(angles, angles)."""
    inv = (1.0 / (np.float32(cfg.rope_theta) ** (np.arange(0, cfg.head_dim, 2, dtype=np.float32) / np.float32(cfg.head_dim)))).astype(np.float32)
    ang = np.arange(cfg.max_cache_len, dtype=np.float32)[:, None] * inv[None, :]
    emb = np.concatenate([ang, ang], axis=1).astype(np.float32)
    return np.cos(emb).astype(np.float32), np.sin(emb).astype(np.float32)


def random_weights(cfg: LlamaConfig, seed: int = 4, sigma: float = 0.02) -> dict:
    """Seeded synthetic weights with the architecture's shapes: every matrix ~ N(0, sigma) drawn from
    numpy.random.default_rng(seed * 1000 + index), norm weights 1."""
    idx = [0]

    def draw(*shape):
        rng = np.random.default_rng(seed * 1000 + idx[0])
        idx[0] += 1
        return (rng.standard_normal(shape) * sigma).astype(np.float32)

    H, I = cfg.hidden_size, cfg.intermediate_size
    w = {"embed": draw(cfg.vocab_size, H), "norm": np.ones(H, dtype=np.float32), "layers": []}
    for _ in range(cfg.num_hidden_layers):
        w["layers"].append({
            "input_norm": np.ones(H, dtype=np.float32), "post_norm": np.ones(H, dtype=np.float32),
            "q": draw(cfg.q_size, H), "k": draw(cfg.kv_size, H), "v": draw(cfg.kv_size, H),
            "q_bias": draw(cfg.q_size), "k_bias": draw(cfg.kv_size), "v_bias": draw(cfg.kv_size),
            "o": draw(H, cfg.q_size), "gate": draw(I, H), "up": draw(I, H), "down": draw(H, I),
        })
    return w


class KvCache:
    """K and V for every layer, [layers][kv_heads][max_len][head_dim], with the per-layer cursor on the device
    (crates/grilly-infer/src/kv_cache.rs:21-33): float32 as the reference's, or with ``int8=True`` int8 codes and one
    float32 scale per cached row (a quarter of the bytes a decoded token reads; no counterpart in the reference)."""

    def __init__(self, cfg: LlamaConfig, int8: bool = False) -> None:
        self.cfg, self.int8 = cfg, bool(int8)
        self.layer_elems = cfg.num_key_value_heads * cfg.max_cache_len * cfg.head_dim
        self.layer_rows = cfg.num_key_value_heads * cfg.max_cache_len
        n = cfg.num_hidden_layers * self.layer_elems
        if self.int8:
            self.k = _C.Tensor.from_numpy(np.zeros(n // 4, dtype=np.int32), persistent=True)  # n bytes of int8 codes
            self.v = _C.Tensor.from_numpy(np.zeros(n // 4, dtype=np.int32), persistent=True)
            rows = cfg.num_hidden_layers * self.layer_rows
            self.kscale = _C.Tensor.from_numpy(np.ones(rows, dtype=np.float32), persistent=True)
            self.vscale = _C.Tensor.from_numpy(np.ones(rows, dtype=np.float32), persistent=True)
        else:
            self.k = _C.Tensor.empty((n,), "float32", persistent=True)
            self.v = _C.Tensor.empty((n,), "float32", persistent=True)
            self.kscale = self.vscale = None
        self.lens = _C.Tensor.from_numpy(np.zeros(cfg.num_hidden_layers, dtype=np.int32), persistent=True)
        out = ctypes.c_uint64()
        check(_lib.load().gq_attn_scratch_bytes(_C.context(), cfg.num_attention_heads, cfg.head_dim, cfg.max_cache_len, ctypes.byref(out)))
        self.scratch = _C.Tensor.from_numpy(np.zeros(out.value // 4, dtype=np.float32), persistent=True)

    def fill(self, k: np.ndarray, v: np.ndarray, length: int) -> None:
        """Install `length` cached positions: k, v are [layers][kv_heads][length][head_dim] (float32 cache only)."""
        if self.int8:
            raise NotImplementedError("grilly: installing float rows into an int8 cache is not implemented yet (prefill instead)")
        c = self.cfg
        full_k = np.zeros((c.num_hidden_layers, c.num_key_value_heads, c.max_cache_len, c.head_dim), dtype=np.float32)
        full_v = np.zeros_like(full_k)
        full_k[:, :, :length], full_v[:, :, :length] = k, v
        self.k = _C.Tensor.from_numpy(full_k.reshape(-1), persistent=True)
        self.v = _C.Tensor.from_numpy(full_v.reshape(-1), persistent=True)
        self.lens = _C.Tensor.from_numpy(np.full(c.num_hidden_layers, length, dtype=np.int32), persistent=True)

    def nbytes(self) -> int:
        per = self.cfg.num_hidden_layers * self.layer_elems
        return 2 * (per + 4 * self.cfg.num_hidden_layers * self.layer_rows) if self.int8 else 2 * 4 * per

    def lengths(self) -> np.ndarray:
        return self.lens.numpy()


class LlamaDecoder:
    """The quantized model and its cache; ``step(token)`` decodes one token."""

    def __init__(self, cfg: LlamaConfig, weights: dict, fused: bool = True, int8_kv: bool = False, persistent: bool = False) -> None:
        self.cfg = cfg
        # persistent: the whole step as one cooperative kernel (gq_decode_plan_*) instead of a launch per operator
        self.persistent = bool(persistent) and not int8_kv
        self._plan = None
        # fused: norms and SwiGLU run inside the following projection (one launch each); needs row lengths that are multiples of 4
        self.fused = fused and cfg.hidden_size % 4 == 0 and cfg.intermediate_size % 4 == 0
        self.int8_kv = bool(int8_kv)
        T = _C.Tensor.from_numpy

        def q8(a):
            return _C.Int8Weight.quantize(T(np.ascontiguousarray(a, dtype=np.float32)))

        def q8_fused(parts):  # q | k | v and gate | up are quantized straight into the fused weight: no second copy of the parts
            return _C.Int8Weight.quantize_fused([T(np.ascontiguousarray(a, dtype=np.float32)) for a in parts])

        self.embed = T(weights["embed"], persistent=True)
        self.lm_head = q8(weights["embed"])  # tied; the table itself stays float32
        self.norm = T(weights["norm"], persistent=True)
        self.layers = []
        for lw in weights["layers"]:
            self.layers.append({
                "input_norm": T(lw["input_norm"], persistent=True), "post_norm": T(lw["post_norm"], persistent=True),
                "qkv": q8_fused([lw["q"], lw["k"], lw["v"]]),
                "qkv_bias": T(np.concatenate([lw["q_bias"], lw["k_bias"], lw["v_bias"]]), persistent=True) if cfg.attention_bias else None,
                "o": q8(lw["o"]),
                "gate_up": q8_fused([lw["gate"], lw["up"]]),
                "down": q8(lw["down"]),
            })
        cos, sin = rotary_tables(cfg)
        self.cos, self.sin = T(cos, persistent=True), T(sin, persistent=True)
        self.cache = KvCache(cfg, int8=self.int8_kv)

    # the operators, as thin calls into the C ABI
    def _norm(self, x, residual, weight, want_sum: bool, rows: int = 1):
        H = self.cfg.hidden_size
        y = _C.Tensor.empty((rows, H), "float32")
        h = _C.Tensor.empty((rows, H), "float32") if want_sum else None
        check(_lib.load().gq_add_rms_norm(_C.context(), x.storage.handle, residual.storage.handle if residual is not None else 0,
                                          weight.storage.handle, rows, H, self.cfg.rms_norm_eps, y.storage.handle,
                                          h.storage.handle if h is not None else 0))
        return y, h

    def _attend_rows(self, qkv, rows: int, li: int):
        """Rotary + cache append + causal attention for `rows` new tokens of layer li (gq_attn_prefill)."""
        c, cache = self.cfg, self.cache
        off = li * cache.layer_elems
        attn = _C.Tensor.empty((rows, c.q_size), "float32")
        q_rot = _C.Tensor.empty((rows, c.q_size), "float32")
        check(_lib.load().gq_attn_prefill(
            _C.context(), qkv.storage.handle, rows, self.cos.storage.handle, self.sin.storage.handle, cache.k.storage.handle, off,
            cache.v.storage.handle, off, cache.kscale.storage.handle if cache.int8 else 0, cache.vscale.storage.handle if cache.int8 else 0,
            cache.lens.storage.handle, li, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads, c.head_dim, c.max_cache_len,
            float(c.head_dim) ** -0.5, q_rot.storage.handle, attn.storage.handle))
        return attn

    def prefill(self, tokens: "_C.Tensor"):
        """tokens: int32 [T], continuing the cache from its cursor. Every layer runs on all T rows at once — the linears
        take the kernel their row count selects (the streaming decode kernels for one or two rows, the integer tensor-core GEMM from three) — with causal
        attention over the cache (python/grilly/infer/models/llama.py:340-366 with logits_to_keep=1). Returns the LAST
        position's logits [1, vocab] and advances the cursor by T."""
        c, lib, ctx = self.cfg, _lib.load(), _C.context()
        T = tokens.numel()
        if T == 0:
            raise RuntimeError("prefill needs at least one token")
        hidden = _C.Tensor.empty((T, c.hidden_size), "float32")
        check(lib.gq_embedding(ctx, self.embed.storage.handle, tokens.storage.handle, T, c.hidden_size, c.vocab_size, hidden.storage.handle))
        delta = None
        for li, lw in enumerate(self.layers):
            x, summed = self._norm(hidden, delta, lw["input_norm"], delta is not None, T)
            if summed is not None:
                hidden = summed
            qkv = lw["qkv"].linear(x, lw["qkv_bias"])
            o = lw["o"].linear(self._attend_rows(qkv, T, li))
            x, hidden = self._norm(hidden, o, lw["post_norm"], True, T)
            gu = lw["gate_up"].linear(x)
            act = _C.Tensor.empty((T, c.intermediate_size), "float32")
            check(lib.gq_swiglu(ctx, gu.storage.handle, T, c.intermediate_size, act.storage.handle))
            delta = lw["down"].linear(act)
        last_h, last_d = hidden.window_rows(T - 1, 1), delta.window_rows(T - 1, 1)
        x, _ = self._norm(last_h, last_d, self.norm, False)
        logits = self.lm_head.linear(x)
        check(lib.gq_kv_advance_by(ctx, self.cache.lens.storage.handle, c.num_hidden_layers, c.max_cache_len, T))
        return logits

    def _make_plan(self):
        c, lib = self.cfg, _lib.load()
        layers = (_lib.DecodeLayer * c.num_hidden_layers)()
        for i, lw in enumerate(self.layers):
            d = layers[i]
            d.input_norm, d.post_norm = lw["input_norm"].storage.handle, lw["post_norm"].storage.handle
            d.qkv_q, d.qkv_scale = lw["qkv"]._qt.storage.handle, lw["qkv"]._scale.storage.handle
            d.qkv_bias = lw["qkv_bias"].storage.handle if lw["qkv_bias"] is not None else 0
            d.o_q, d.o_scale = lw["o"]._qt.storage.handle, lw["o"]._scale.storage.handle
            d.gate_up_q, d.gate_up_scale = lw["gate_up"]._qt.storage.handle, lw["gate_up"]._scale.storage.handle
            d.down_q, d.down_scale = lw["down"]._qt.storage.handle, lw["down"]._scale.storage.handle
        desc = _lib.DecodeDesc(hidden=c.hidden_size, heads=c.num_attention_heads, kv_heads=c.num_key_value_heads, dim=c.head_dim,
                               inter=c.intermediate_size, vocab=c.vocab_size, layers=c.num_hidden_layers, max_len=c.max_cache_len,
                               eps=c.rms_norm_eps, attn_scale=float(c.head_dim) ** -0.5, embed=self.embed.storage.handle,
                               final_norm=self.norm.storage.handle, head_q=self.lm_head._qt.storage.handle,
                               head_scale=self.lm_head._scale.storage.handle, cos=self.cos.storage.handle, sin=self.sin.storage.handle,
                               kcache=self.cache.k.storage.handle, vcache=self.cache.v.storage.handle, lens=self.cache.lens.storage.handle,
                               layer=layers)
        out = ctypes.c_void_p()
        check(lib.gq_decode_plan_create(_C.context(), ctypes.byref(desc), ctypes.byref(out)))
        self._plan, self._plan_cache = out, (self.cache.k, self.cache.v, self.cache.lens)

    def __del__(self):
        try:
            if self._plan is not None:
                _lib.load().gq_decode_plan_destroy(_C.context(), self._plan)
        except Exception:
            pass

    def step(self, token: "_C.Tensor", want_argmax: bool = True):
        """token: int32 [1]. Returns (logits [1, vocab], next_token int32 [1]); advances the cache. With want_argmax
        False the greedy token is not computed (a sampler follows) and None is returned in its place."""
        c, lib, ctx = self.cfg, _lib.load(), _C.context()
        if self.persistent:
            if self._plan is None or self._plan_cache[0] is not self.cache.k or self._plan_cache[2] is not self.cache.lens:
                if self._plan is not None:
                    lib.gq_decode_plan_destroy(ctx, self._plan)
                self._make_plan()  # names the cache's buffers: made anew when fill() replaced them
            logits = _C.Tensor.empty((1, c.vocab_size), "float32")
            nxt = _C.Tensor.empty((1,), "int32")
            check(lib.gq_decode_plan_step(ctx, self._plan, token.storage.handle, logits.storage.handle, nxt.storage.handle))
            return logits, nxt
        L, Hq, Hkv, D = c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads, c.head_dim
        hidden = _C.Tensor.empty((1, c.hidden_size), "float32")
        check(lib.gq_embedding(ctx, self.embed.storage.handle, token.storage.handle, 1, c.hidden_size, c.vocab_size, hidden.storage.handle))
        delta = None  # what the last block produced; added to `hidden` by the next norm
        fused = self.fused
        for li, lw in enumerate(self.layers):
            if fused:  # the norm runs inside the projection's conversion of its input row
                qkv, summed = lw["qkv"].linear_norm(hidden, delta, lw["input_norm"], c.rms_norm_eps, lw["qkv_bias"], delta is not None)
            else:
                x, summed = self._norm(hidden, delta, lw["input_norm"], delta is not None)
                qkv = lw["qkv"].linear(x, lw["qkv_bias"])
            if summed is not None:
                hidden = summed
            off = li * self.cache.layer_elems
            attn = _C.Tensor.empty((1, c.q_size), "float32")
            if self.int8_kv:  # the int8 cache: rotary, quantized append and attention through the prompt kernels, one row
                attn = self._attend_rows(qkv, 1, li)
            elif fused:  # rotary, the cache append and attention in one launch
                check(lib.gq_attn_decode_rope(ctx, qkv.storage.handle, self.cos.storage.handle, self.sin.storage.handle,
                                              self.cache.k.storage.handle, off, self.cache.v.storage.handle, off,
                                              self.cache.lens.storage.handle, li, L, Hq, Hkv, D, c.max_cache_len, float(D) ** -0.5,
                                              self.cache.scratch.storage.handle, attn.storage.handle))
            else:
                q = _C.Tensor.empty((1, c.q_size), "float32")
                check(lib.gq_rope_kv_append(ctx, qkv.storage.handle, self.cos.storage.handle, self.sin.storage.handle,
                                            self.cache.lens.storage.handle, li, L, Hq, Hkv, D, c.max_cache_len, q.storage.handle,
                                            self.cache.k.storage.handle, off, self.cache.v.storage.handle, off))
                check(lib.gq_attn_decode(ctx, q.storage.handle, self.cache.k.storage.handle, off, self.cache.v.storage.handle, off,
                                         self.cache.lens.storage.handle, li, L, Hq, Hkv, D, c.max_cache_len, float(D) ** -0.5,
                                         self.cache.scratch.storage.handle, attn.storage.handle))
            o = lw["o"].linear(attn)
            if fused:
                gu, hidden = lw["gate_up"].linear_norm(hidden, o, lw["post_norm"], c.rms_norm_eps, None, True)
                delta = lw["down"].linear_swiglu(gu)
            else:
                x, hidden = self._norm(hidden, o, lw["post_norm"], True)
                gu = lw["gate_up"].linear(x)
                act = _C.Tensor.empty((1, c.intermediate_size), "float32")
                check(lib.gq_swiglu(ctx, gu.storage.handle, 1, c.intermediate_size, act.storage.handle))
                delta = lw["down"].linear(act)
        if fused:
            logits, _ = self.lm_head.linear_norm(hidden, delta, self.norm, c.rms_norm_eps)
        else:
            x, _ = self._norm(hidden, delta, self.norm, False)
            logits = self.lm_head.linear(x)
        nxt = None
        if want_argmax:
            nxt = _C.Tensor.empty((1,), "int32")
            check(lib.gq_argmax_rows(ctx, logits.storage.handle, 1, c.vocab_size, nxt.storage.handle))
        check(lib.gq_kv_advance(ctx, self.cache.lens.storage.handle, L, c.max_cache_len))
        return logits, nxt

    def bytes_per_token(self) -> dict:
        """Algorithmic bytes one decode step touches at the cache's current length."""
        c = self.cfg
        lin = sum(sum(lw[k].nbytes for k in ("qkv", "o", "gate_up", "down")) for lw in self.layers) + self.lm_head.nbytes
        kv = 2 * c.num_hidden_layers * c.num_key_value_heads * c.max_cache_len * c.head_dim * 4
        other = 4 * (c.vocab_size + 40 * c.hidden_size * c.num_hidden_layers)
        return {"linear_weights": lin, "kv_cache_at_full_length": kv, "other": other, "total": lin + kv + other}
