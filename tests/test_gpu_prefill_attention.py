"""Prompt processing (gq_attn_prefill, LlamaDecoder.prefill) and the int8 KV cache on a GPU against the float64 numpy
model (oracle/llama_ref.py) stepping through the same tokens one by one — causal attention over a prompt equals
decoding it token by token.

Tolerances: prompts of fewer than 64 tokens run every linear on the decode kernels, so the last position's logits are
held to the decode step's 1e-5 * max|logit|; from 64 tokens the linears are the tf32 tensor-core GEMM, held to its
2e-3. The int8 cache is lossy by construction (one scale per cached row, 127 levels): it is compared with the oracle
applying the same storage rule, to 5e-3 * max|logit| (a code that falls on a rounding boundary may differ by one).
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def small_config(max_len=128):
    from grilly2_b200.infer.llama import LlamaConfig
    return LlamaConfig(vocab_size=500, hidden_size=128, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
                       head_dim=32, intermediate_size=256, max_cache_len=max_len)


def build(seed, int8_kv=False, max_len=128):
    from grilly2_b200.infer import llama
    from oracle.llama_ref import DecoderRef
    cfg = small_config(max_len)
    w = llama.random_weights(cfg, seed=seed, sigma=0.06)
    cos, sin = llama.rotary_tables(cfg)
    return cfg, llama.LlamaDecoder(cfg, w, int8_kv=int8_kv), DecoderRef(cfg, w, cos, sin, int8_kv=int8_kv)


def worst(got, want, what):
    ratio = float(np.abs(got - want).max() / np.abs(want).max())
    print(f"[prefill parity] {what}: max|logit - ref| / max|ref| = {ratio:.3e}")
    return ratio


def tokens_of(n, seed=0):
    return np.random.default_rng(seed).integers(0, 500, n).astype(np.int32)


@pytest.mark.parametrize("chunks", [(12,), (5, 7), (1, 11), (16, 3)], ids=["whole", "5+7", "1+11", "16+3"])
def test_prefill_equals_decoding_the_prompt_token_by_token(chunks):
    from grilly2_b200 import _C
    cfg, model, ref = build(11)
    toks = tokens_of(sum(chunks))
    for t in toks:
        want = ref.step(int(t))
    at = 0
    for n in chunks:
        logits = model.prefill(_C.Tensor.from_numpy(toks[at:at + n]))
        at += n
    assert worst(logits.numpy()[0], want, f"prompt in chunks {chunks}") <= 1e-5
    assert (model.cache.lengths() == len(toks)).all()
    # and a decode step continues from there
    logits, nxt = model.step(_C.Tensor.from_numpy(np.array([7], dtype=np.int32)))
    want = ref.step(7)
    assert worst(logits.numpy()[0], want, "the step after the prompt") <= 1e-5
    assert int(nxt.numpy()[0]) == int(np.argmax(want))


def test_a_long_prompt_runs_the_tensor_core_linears_within_their_tolerance():
    from grilly2_b200 import _C
    cfg, model, ref = build(12)
    toks = tokens_of(80, 1)
    for t in toks:
        want = ref.step(int(t))
    logits = model.prefill(_C.Tensor.from_numpy(toks))
    assert worst(logits.numpy()[0], want, "80-token prompt (tf32 linears)") <= 2e-3
    assert (model.cache.lengths() == 80).all()


def test_int8_kv_cache_follows_the_same_storage_rule_as_the_oracle_and_is_a_quarter_of_the_bytes():
    from grilly2_b200 import _C
    cfg, model, ref = build(13, int8_kv=True)
    _, float_model, _ = build(13)
    assert model.cache.nbytes() * 3 < float_model.cache.nbytes()  # dim codes + one float32 scale per row of 32
    toks = tokens_of(10, 2)
    for t in toks:
        want = ref.step(int(t))
    logits = model.prefill(_C.Tensor.from_numpy(toks))
    assert worst(logits.numpy()[0], want, "int8 cache, 10-token prompt") <= 5e-3
    tok = 9
    for step in range(3):
        logits, nxt = model.step(_C.Tensor.from_numpy(np.array([tok], dtype=np.int32)))
        want = ref.step(tok)
        assert worst(logits.numpy()[0], want, f"int8 cache, decode step {step}") <= 5e-3
        tok = int(np.argmax(want))
    assert (model.cache.lengths() == 13).all()


@pytest.mark.parametrize("dim,heads,kv_heads", [(32, 4, 2), (64, 14, 2), (128, 8, 8)])
def test_attention_kernel_alone_against_numpy(dim, heads, kv_heads):
    """gq_attn_prefill on random rows over a part-filled cache, all three head sizes, against float64."""
    import ctypes
    from grilly2_b200 import _C, _lib
    lib, ctx = _lib.load(), _C.context()
    rng = np.random.default_rng(dim)
    max_len, filled, rows = 96, 37, 9
    qkv = rng.standard_normal((rows, (heads + 2 * kv_heads) * dim)).astype(np.float32)
    kc = rng.standard_normal((kv_heads, max_len, dim)).astype(np.float32)
    vc = rng.standard_normal((kv_heads, max_len, dim)).astype(np.float32)
    ang = rng.standard_normal((max_len, dim)).astype(np.float32)
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    T = _C.Tensor.from_numpy
    tq, tk, tv, tc, ts = T(qkv), T(kc.reshape(-1)), T(vc.reshape(-1)), T(cos), T(sin)
    lens = T(np.array([filled], dtype=np.int32))
    qs, out = _C.Tensor.empty((rows, heads * dim), "float32"), _C.Tensor.empty((rows, heads * dim), "float32")
    _lib.check(lib.gq_attn_prefill(ctx, tq.storage.handle, rows, tc.storage.handle, ts.storage.handle, tk.storage.handle, 0, tv.storage.handle, 0,
                                   0, 0, lens.storage.handle, 0, 1, heads, kv_heads, dim, max_len, dim ** -0.5, qs.storage.handle, out.storage.handle))
    got = out.numpy().astype(np.float64)

    def rope(x, pos):
        x = x.reshape(-1, dim).astype(np.float64)
        rot = np.concatenate([-x[:, dim // 2:], x[:, :dim // 2]], axis=1)
        return x * cos[pos].astype(np.float64) + rot * sin[pos].astype(np.float64)

    K, V = kc.astype(np.float64).copy(), vc.astype(np.float64).copy()
    for t in range(rows):
        K[:, filled + t] = rope(qkv[t, heads * dim:(heads + kv_heads) * dim], filled + t)
        V[:, filled + t] = qkv[t, (heads + kv_heads) * dim:].reshape(kv_heads, dim)
    rep = heads // kv_heads
    for t in range(rows):
        q = rope(qkv[t, :heads * dim], filled + t)
        n = filled + t + 1
        for h in range(heads):
            s = K[h // rep, :n] @ q[h] / np.sqrt(dim)
            e = np.exp(s - s.max())
            want = (e / e.sum()) @ V[h // rep, :n]
            assert np.abs(got[t, h * dim:(h + 1) * dim] - want).max() <= 2e-6 * max(np.abs(want).max(), 1.0)
    np.testing.assert_allclose(tk.numpy().reshape(kv_heads, max_len, dim)[:, filled:filled + rows], K[:, filled:filled + rows], rtol=0, atol=2e-6)
