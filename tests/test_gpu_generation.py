"""generate() over the int8 decoder on a GPU: greedy against the float64 numpy model decoding greedily (as
tests/python/test_generation.py:66-72 holds the reference to transformers' greedy output), end-of-sequence stopping,
sampling determinism, and the captured loop equal to the eager one."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def small_config():
    from grilly2_b200.infer.llama import LlamaConfig
    return LlamaConfig(vocab_size=500, hidden_size=128, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
                       head_dim=32, intermediate_size=256, max_cache_len=64)


def build(seed):
    from grilly2_b200.infer import llama
    from oracle.llama_ref import DecoderRef
    cfg = small_config()
    w = llama.random_weights(cfg, seed=seed, sigma=0.08)
    cos, sin = llama.rotary_tables(cfg)
    return cfg, w, (lambda: llama.LlamaDecoder(cfg, w)), DecoderRef(cfg, w, cos, sin)


PROMPT = [5, 17, 99, 3, 42, 7, 64]


@pytest.mark.parametrize("graphed", [True, False], ids=["graphed", "eager"])
def test_greedy_generate_matches_the_float64_model(graphed):
    from grilly2_b200.infer.generation import generate
    cfg, w, make, ref = build(1)
    want = list(PROMPT)
    for t in PROMPT[:-1]:
        ref.step(t)
    tok = PROMPT[-1]
    for _ in range(16):
        tok = int(np.argmax(ref.step(tok)))
        want.append(tok)
    got = generate(make(), np.array([PROMPT]), max_new_tokens=16, do_sample=False, graphed=graphed)
    assert got.dtype == np.int64 and got.shape == (1, len(PROMPT) + 16)
    assert got[0].tolist() == want
    assert len(set(want[len(PROMPT):])) > 3  # the weights give varied tokens, so this compares something


def test_eos_stops_the_sequence_and_max_length_counts_the_prompt():
    from grilly2_b200.infer.generation import generate
    cfg, w, make, _ = build(2)
    free = generate(make(), np.array([PROMPT]), max_new_tokens=10)[0].tolist()
    eos = free[len(PROMPT) + 3]
    stopped = generate(make(), np.array([PROMPT]), max_new_tokens=10, eos_token_id=eos)[0].tolist()
    cut = free.index(eos, len(PROMPT))
    assert stopped == free[:cut + 1]
    assert generate(make(), PROMPT, max_length=len(PROMPT) + 2).shape == (1, len(PROMPT) + 2)
    assert generate(make(), PROMPT, max_length=3).tolist() == [PROMPT]  # nothing to add


def test_sampling_is_seeded_graph_equals_eager_and_respects_top_k():
    from grilly2_b200.infer.generation import generate
    from grilly2_b200.infer.sampling import Generator
    cfg, w, make, ref = build(3)
    kw = dict(max_new_tokens=12, do_sample=True, temperature=0.9, top_k=5, top_p=0.95, repetition_penalty=1.1)
    a = generate(make(), PROMPT, generator=Generator(7), **kw)[0].tolist()
    b = generate(make(), PROMPT, generator=Generator(7), graphed=False, **kw)[0].tolist()
    c = generate(make(), PROMPT, generator=Generator(8), **kw)[0].tolist()
    assert a == b and a != c
    # every sampled token is among the five most likely of its step (before the penalty reorders little at 1.1: allow ten)
    for t in PROMPT[:-1]:
        ref.step(t)
    tok = PROMPT[-1]
    for got in a[len(PROMPT):]:
        logits = ref.step(tok)
        assert got in np.argsort(logits)[-10:]
        tok = got


def test_refusals_name_what_is_wrong():
    from grilly2_b200.infer.generation import generate
    cfg, w, make, _ = build(4)
    with pytest.raises(ValueError, match="not used by the model"):
        generate(make(), PROMPT, max_new_tokens=2, banana=1)
    with pytest.raises(NotImplementedError, match="num_beams"):
        generate(make(), PROMPT, max_new_tokens=2, num_beams=4)
    with pytest.raises(ValueError, match="needs `inputs`"):
        generate(make())
