"""The decode step of the int8 weight-only Llama/Qwen2 decoder on a GPU against
the float64 numpy model (oracle/llama_ref.py), mirroring
tests/python/test_generation.py:46-70 and test_fused_ops.py of the reference.

Tolerance: |logits - ref| <= TOL * max|ref| against float64, with TOL the
reference's own 1e-5 (tests/python/test_generation.py:53,58 holds its float32
model to that against another float32 implementation) on the path made of the
separate operators, and TOL_FUSED on the path whose SwiGLU runs inside the
GEMV's prologue with the hardware exp2 / reciprocal. Each test prints the worst
ratio it saw, so the margin is on record. Greedy tokens identical, and a graph
replay equal to the eager step bit for bit.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 1e-5        # the separate operators: the reference's own bound
TOL_FUSED = 1e-5  # norm, SwiGLU and rotary fused into their neighbours


def worst(got, want, what):
    ratio = float(np.abs(got - want).max() / np.abs(want).max())
    print(f"[decode parity] {what}: max|logit - ref| / max|ref| = {ratio:.3e}")
    return ratio


def small_config():
    from grilly2_b200.infer.llama import LlamaConfig
    return LlamaConfig(vocab_size=500, hidden_size=128, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
                       head_dim=32, intermediate_size=256, max_cache_len=48)


def build(cfg, seed, prefill, fused=True, persistent=False):
    from grilly2_b200.infer import llama
    from oracle.llama_ref import DecoderRef
    w = llama.random_weights(cfg, seed=seed, sigma=0.05)
    for i, lw in enumerate(w["layers"]):  # non-trivial norm weights
        lw["input_norm"] = (1 + 0.1 * np.random.default_rng(100 + i).standard_normal(cfg.hidden_size)).astype(np.float32)
    model = llama.LlamaDecoder(cfg, w, fused=fused, persistent=persistent)
    cos, sin = llama.rotary_tables(cfg)
    ref = DecoderRef(cfg, w, cos, sin)
    if prefill:
        rng = np.random.default_rng(9)
        shape = (cfg.num_hidden_layers, cfg.num_key_value_heads, prefill, cfg.head_dim)
        k, v = rng.standard_normal(shape).astype(np.float32), rng.standard_normal(shape).astype(np.float32)
        model.cache.fill(k, v, prefill)
        ref.fill(k, v, prefill)
    return model, ref


@pytest.mark.parametrize("prefill,fused", [(0, True), (20, True), (20, False)])
def test_decode_steps_match_the_float64_model(prefill, fused):
    from grilly2_b200 import _C
    cfg = small_config()
    model, ref = build(cfg, 4, prefill, fused)
    assert model.fused == fused
    token = 7
    for step in range(4):
        logits, nxt = model.step(_C.Tensor.from_numpy(np.array([token], dtype=np.int32)))
        want = ref.step(token)
        got = logits.numpy()[0]
        assert worst(got, want, f"small model, prefill {prefill}, fused {fused}, step {step}") <= (TOL_FUSED if fused else TOL), f"step {step}"
        assert int(nxt.numpy()[0]) == int(np.argmax(want))
        assert (model.cache.lengths() == prefill + step + 1).all()
        token = int(nxt.numpy()[0])


def test_a_full_cache_saturates():
    from grilly2_b200 import _C
    cfg = small_config()
    model, _ = build(cfg, 5, cfg.max_cache_len - 1)
    t = _C.Tensor.from_numpy(np.array([3], dtype=np.int32))
    model.step(t)
    assert (model.cache.lengths() == cfg.max_cache_len).all()
    logits, _ = model.step(t)  # nothing more is appended; the step still answers
    assert np.isfinite(logits.numpy()).all() and (model.cache.lengths() == cfg.max_cache_len).all()


def test_captured_step_replays_like_the_eager_one():
    """First call eager, second captured, later ones replayed: the position comes from the device cursor, so
    a replay rotates q and k at the right place (the reference's step would bake a host integer in)."""
    import grilly2_b200 as g
    from grilly2_b200 import _C
    cfg = small_config()
    eager, _ = build(cfg, 6, 10)
    fast_model, _ = build(cfg, 6, 10)
    fast = g.graphed(fast_model.step)
    tokens = [5, 9, 11, 2, 40, 41]
    for tk in tokens:
        t = np.array([tk], dtype=np.int32)
        le, ne = eager.step(_C.Tensor.from_numpy(t))
        lf, nf = fast(_C.Tensor.from_numpy(t))
        np.testing.assert_array_equal(lf.numpy(), le.numpy())
        assert int(nf.numpy()[0]) == int(ne.numpy()[0])
    assert (fast.misses, fast.captures, fast.replays) == (1, 1, 4)
    assert (fast_model.cache.lengths() == 10 + len(tokens)).all()


@pytest.mark.parametrize("fused", [True, False], ids=["fused", "separate"])
def test_full_size_config5_step(fused):
    """Qwen2.5-0.5B architecture, cache pre-filled to 1023 positions, one step at position 1023."""
    from grilly2_b200 import _C
    from grilly2_b200.infer import llama
    cfg = llama.qwen25_05b(1024)
    model, ref = build(cfg, 4, 1023, fused)
    logits, nxt = model.step(_C.Tensor.from_numpy(np.array([12345], dtype=np.int32)))
    want = ref.step(12345)
    got = logits.numpy()[0]
    assert worst(got, want, f"config 5, fused {fused}") <= (TOL_FUSED if fused else TOL)
    assert int(nxt.numpy()[0]) == int(np.argmax(want))
    assert (model.cache.lengths() == 1024).all()


@pytest.mark.parametrize("prefill", [0, 20, 47])
def test_the_persistent_step_matches_the_float64_model_and_the_operator_by_operator_step(prefill):
    """One cooperative kernel for the whole step: same tolerance against float64 as the launch-per-operator step, the
    same greedy tokens, the same cache contents, and (captured) the same results when replayed."""
    import grilly2_b200 as g
    from grilly2_b200 import _C
    cfg = small_config()
    model, ref = build(cfg, 4, prefill, persistent=True)
    twin, _ = build(cfg, 4, prefill)
    token = 7
    for step in range(min(4, cfg.max_cache_len - prefill)):  # up to the cache's last position (a full cache is the next test's)
        t = _C.Tensor.from_numpy(np.array([token], dtype=np.int32))
        logits, nxt = model.step(t)
        lt, nt = twin.step(t)
        want = ref.step(token)
        got = logits.numpy()[0]
        assert worst(got, want, f"persistent step, prefill {prefill}, step {step}") <= TOL
        assert np.abs(got - lt.numpy()[0]).max() <= 2e-6 * np.abs(want).max()
        assert int(nxt.numpy()[0]) == int(np.argmax(want)) == int(nt.numpy()[0])
        np.testing.assert_array_equal(model.cache.lengths(), twin.cache.lengths())
        token = int(nxt.numpy()[0])
    # the positions written so far (the rest of a cache is uninitialised memory)
    filled = int(model.cache.lengths()[0])
    shape = (cfg.num_hidden_layers, cfg.num_key_value_heads, cfg.max_cache_len, cfg.head_dim)
    for mine, theirs in ((model.cache.k, twin.cache.k), (model.cache.v, twin.cache.v)):
        np.testing.assert_allclose(mine.numpy().reshape(shape)[:, :, :filled], theirs.numpy().reshape(shape)[:, :, :filled], rtol=0, atol=2e-6)


def test_the_persistent_step_replays_in_a_graph_and_saturates_a_full_cache():
    import grilly2_b200 as g
    from grilly2_b200 import _C
    cfg = small_config()
    eager, _ = build(cfg, 6, 40, persistent=True)
    fast_model, _ = build(cfg, 6, 40, persistent=True)
    fast = g.graphed(fast_model.step)
    for tk in [5, 9, 11, 2, 40, 41, 3, 8, 1, 2]:  # ten steps from 40: the cache (48) fills up on the way
        t = np.array([tk], dtype=np.int32)
        le, ne = eager.step(_C.Tensor.from_numpy(t))
        lf, nf = fast(_C.Tensor.from_numpy(t))
        np.testing.assert_array_equal(lf.numpy(), le.numpy())
        assert int(nf.numpy()[0]) == int(ne.numpy()[0])
    assert (fast.misses, fast.captures, fast.replays) == (1, 1, 8)
    assert (fast_model.cache.lengths() == cfg.max_cache_len).all()


def test_full_size_config5_persistent_step():
    from grilly2_b200 import _C
    from grilly2_b200.infer import llama
    cfg = llama.qwen25_05b(1024)
    model, ref = build(cfg, 4, 1023, persistent=True)
    logits, nxt = model.step(_C.Tensor.from_numpy(np.array([12345], dtype=np.int32)))
    want = ref.step(12345)
    assert worst(logits.numpy()[0], want, "config 5, persistent") <= TOL
    assert int(nxt.numpy()[0]) == int(np.argmax(want))
    assert (model.cache.lengths() == 1024).all()
