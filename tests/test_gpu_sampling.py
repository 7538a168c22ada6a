"""Device-side next-token selection (gq_sample) against Hugging Face's own logits processors (transformers, run in
torch on the CPU), mirroring tests/python/test_sampling.py of the reference.

Tolerances, as that file states them:
- kept tokens after top-k: identical;
- kept tokens after top-p: identical, except that a token whose cumulative probability (HF's ascending cumsum) is
  within 1e-6 of 1 - top_p may be decided differently (HF sums sorted float32 probabilities in order, the kernel sums
  masses in a tree), and among tokens tied at the cut only the COUNT must match (torch.sort orders ties unstably);
- probabilities: against a float64 softmax of HF's processed scores over the kept tokens, within
  (|x - max| + 8) * 2^-24 relative per token;
- the draw: the token whose float64 CDF interval (in token order, over the kernel's kept set) holds u, or its
  neighbour when u * total is within 1e-6 * total of the boundary;
- many draws: a chi-square goodness-of-fit at the p = 1e-4 quantile with a fixed seed.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

RNG = np.random.default_rng(11)


def hf_scores(logits, ids, *, temperature=1.0, top_k=0, top_p=1.0, penalty=1.0, do_sample=True):
    import torch
    from transformers.generation.logits_process import (LogitsProcessorList, RepetitionPenaltyLogitsProcessor, TemperatureLogitsWarper,
                                                        TopKLogitsWarper, TopPLogitsWarper)
    procs = []
    if penalty != 1.0:
        procs.append(RepetitionPenaltyLogitsProcessor(penalty))
    if do_sample:
        if temperature != 1.0:
            procs.append(TemperatureLogitsWarper(temperature))
        if top_k:
            procs.append(TopKLogitsWarper(top_k))
        if top_p < 1.0:
            procs.append(TopPLogitsWarper(top_p))
    return LogitsProcessorList(procs)(torch.from_numpy(ids.astype(np.int64)), torch.from_numpy(logits.copy())).numpy()


def case(batch, vocab, scale=3.0, history=24):
    return (RNG.standard_normal((batch, vocab)) * scale).astype(np.float32), RNG.integers(0, vocab, (batch, history))


def compare(logits, ids, **kw):
    """The kernel's filtered distribution against HF's; returns how many top-p boundary tokens were decided differently."""
    import torch
    from grilly2_b200 import _C
    from grilly2_b200.infer import sampling
    hf = hf_scores(logits, ids, **kw)
    hf_kept = np.isfinite(hf)
    got = sampling.probabilities(_C.Tensor.from_numpy(logits), ids, temperature=kw.get("temperature", 1.0), top_k=kw.get("top_k", 0),
                                 top_p=kw.get("top_p", 1.0), repetition_penalty=kw.get("penalty", 1.0)).numpy()
    kept = got > 0
    boundary = 0
    before_top_p = hf_scores(logits, ids, **{**kw, "top_p": 1.0})
    for r in np.nonzero((hf_kept != kept).any(1))[0]:
        assert kw.get("top_p", 1.0) < 1.0, "top-k alone must keep exactly HF's tokens"
        differ = hf_kept[r] != kept[r]
        if len(set(before_top_p[r][differ])) == 1 and hf_kept[r].sum() == kept[r].sum():
            continue  # the same number of tokens tied at the cut; torch.sort picks which
        before = torch.from_numpy(before_top_p[r:r + 1])
        order = torch.sort(before, -1).indices
        cum = torch.zeros_like(before).scatter_(1, order, torch.softmax(before, -1).gather(1, order).cumsum(-1))[0]
        gap = np.abs(cum.numpy()[differ] - (1 - kw["top_p"]))
        assert (gap < 1e-6).all(), f"row {r}: tokens decided differently away from the top-p boundary: {gap}"
        boundary += int(differ.sum())
    x = np.where(kept, hf_scores(logits, ids, **{**kw, "top_k": 0, "top_p": 1.0}), -np.inf).astype(np.float64)
    m = x.max(1, keepdims=True)
    e = np.exp(x - m)
    ref = e / e.sum(1, keepdims=True)
    bound = (np.abs(np.where(kept, x - m, 0)) + 8) * 2.0 ** -24 * ref
    ratio = np.abs(got - ref)[kept] / bound[kept]
    assert (ratio <= 1).all(), f"probability error {ratio.max():.2f} x its bound"
    assert (got[~kept] == 0).all()
    return boundary


@pytest.mark.parametrize("vocab", [997, 151936], ids=["small", "qwen-vocab"])
@pytest.mark.parametrize("top_k,top_p", [(0, 1.0), (1, 1.0), (20, 1.0), (50, 0.8), (20, 0.8), (0, 0.9), (0, 0.5), (0, 0.0), (5000, 0.95)])
def test_filtered_distribution_is_hfs(vocab, top_k, top_p):
    boundary = 0
    for penalty, temperature in [(1.0, 1.0), (1.05, 0.7), (1.3, 1.5)]:
        logits, ids = case(3, vocab)
        boundary += compare(logits, ids, temperature=temperature, top_k=top_k, top_p=top_p, penalty=penalty)
    assert boundary <= 1, f"{boundary} top-p boundary tokens decided differently"


def test_ties_and_masked_logits_follow_hf():
    logits, ids = case(2, 300)
    logits[:, :40] = 5.0          # 40 tied maxima: top_k = 20 keeps all of them, as torch.topk's threshold does
    logits[:, 100:200] = -np.inf  # masked, as a suppression processor leaves them
    compare(logits, ids, top_k=20)
    compare(logits, ids, top_k=250, top_p=0.9)
    compare(logits, ids, top_p=0.3)


def test_greedy_is_the_first_index_of_the_maximum_after_the_penalty():
    from grilly2_b200 import _C
    from grilly2_b200.infer import sampling
    logits, ids = case(4, 500)
    logits[0, [7, 300]] = 50.0  # a tie: the first index wins, as torch.argmax
    for penalty in (1.0, 1.4):
        want = hf_scores(logits, ids, penalty=penalty, do_sample=False).argmax(-1)
        got = sampling.next_token(_C.Tensor.from_numpy(logits), ids, repetition_penalty=penalty).numpy()
        np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("vocab,top_k,top_p", [(997, 0, 1.0), (997, 50, 0.9), (151936, 50, 0.8), (151936, 0, 0.95), (5000, 0, 1.0)])
def test_the_draw_is_the_inverse_cdf_in_token_order(vocab, top_k, top_p):
    from grilly2_b200 import _C
    from grilly2_b200.infer import sampling
    rows = 6
    logits, ids = case(rows, vocab)
    kw = dict(temperature=0.8, top_k=top_k, top_p=top_p, repetition_penalty=1.1)
    probs = sampling.probabilities(_C.Tensor.from_numpy(logits), ids, **kw).numpy().astype(np.float64)
    u = sampling.Generator(77).uniform((1, rows))[0].astype(np.float64)
    got = sampling.next_token(_C.Tensor.from_numpy(logits), ids, do_sample=True, generator=sampling.Generator(77), **kw).numpy()
    for r in range(rows):
        cdf = np.cumsum(probs[r])
        target = u[r] * cdf[-1]
        want = int(np.searchsorted(cdf, target, side="right"))
        live = np.nonzero(probs[r] > 0)[0]
        want = int(live[np.searchsorted(live, want)]) if want not in live else want
        if got[r] != want:  # only where u falls on a boundary to within float32 rounding of the running sum
            lo = cdf[got[r]] - probs[r][got[r]]
            assert probs[r][got[r]] > 0 and lo - 1e-6 <= target <= cdf[got[r]] + 1e-6, (r, got[r], want)


def chi2_threshold(dof, z=3.719):
    return dof * (1 - 2 / (9 * dof) + z * (2 / (9 * dof)) ** 0.5) ** 3


@pytest.mark.parametrize("top_k,top_p", [(0, 1.0), (10, 1.0), (0, 0.7)])
def test_draws_follow_the_distribution(top_k, top_p):
    from grilly2_b200 import _C
    from grilly2_b200.infer import sampling
    vocab, rows = 20, 20000
    logits = np.tile(RNG.standard_normal(vocab).astype(np.float32), (rows, 1))
    kw = dict(temperature=0.8, top_k=top_k, top_p=top_p)
    probs = sampling.probabilities(_C.Tensor.from_numpy(logits[:1]), **kw).numpy()[0]
    tokens = sampling.next_token(_C.Tensor.from_numpy(logits), do_sample=True, generator=sampling.Generator(1234), **kw).numpy()
    counts = np.bincount(tokens, minlength=vocab)
    live = probs > 0
    assert counts[~live].sum() == 0, "drew a token with zero probability"
    expected = rows * probs[live]
    stat, dof = float(((counts[live] - expected) ** 2 / expected).sum()), int(live.sum()) - 1
    assert stat < chi2_threshold(dof), f"chi-square {stat:.1f} with {dof} degrees of freedom"


def test_rows_with_nothing_to_draw_give_minus_one_and_validation_is_hfs():
    from grilly2_b200 import _C
    from grilly2_b200.infer import sampling
    dead = _C.Tensor.from_numpy(np.full((3, 151936), -np.inf, np.float32))
    for kw in (dict(), dict(top_k=0, top_p=0.9), dict(top_k=20, top_p=0.5, temperature=0.7)):
        assert sampling.next_token(dead, do_sample=True, **kw).numpy().tolist() == [-1, -1, -1]
    assert sampling.next_token(dead).numpy().tolist() == [0, 0, 0]  # greedy: the first index, as torch.argmax
    x = _C.Tensor.from_numpy(np.zeros((1, 10), np.float32))
    with pytest.raises(RuntimeError, match="strictly positive float"):
        sampling.next_token(x, repetition_penalty=0.0)
    with pytest.raises(RuntimeError, match="temperature"):
        sampling.next_token(x, do_sample=True, temperature=0.0)
    with pytest.raises(RuntimeError, match="top_p"):
        sampling.next_token(x, do_sample=True, top_p=1.5)
    assert sampling.next_token(x, temperature=0.0).numpy().tolist() == [0]  # greedy ignores the sampling fields, as HF


def test_a_captured_sampler_takes_the_next_uniform_and_appends_at_every_replay():
    """The draw counter and the history length live on the device: a graph holding one sampler launch, replayed, uses
    uniform number 0, 1, 2, ... and appends its token to the history each time - no host value is baked in."""
    from grilly2_b200 import _C
    from grilly2_b200.infer import sampling
    vocab, steps = 64, 12
    logits_np = (RNG.standard_normal((1, vocab)) * 2).astype(np.float32)
    logits = _C.Tensor.from_numpy(logits_np, persistent=True)
    kw = dict(do_sample=True, temperature=0.9, top_k=0, top_p=1.0)
    s = sampling.Sampler(1, vocab, history_capacity=steps + 2, draws=steps + 2, generator=sampling.Generator(5), **kw)
    out = _C.Tensor.empty((1,), "int32", persistent=True)
    s.sample(logits, out=out)  # eager: draw 0
    first = int(out.numpy()[0])
    _C.begin_capture()
    s.sample(logits, out=out)
    graph = _C.end_capture()  # the capture runs once: draw 1
    for _ in range(steps - 2):
        graph.replay()
    _C.synchronize()
    hist = s.history.numpy()[0]
    assert int(s.hist_len.numpy()[0]) == steps and int(s.draw_count.numpy()[0]) == steps and hist[0] == first
    # every token is what a one-shot call with that uniform number gives
    u = sampling.Generator(5).uniform((steps + 2, 1))
    probs = sampling.probabilities(logits, temperature=0.9).numpy()[0].astype(np.float64)
    cdf = np.cumsum(probs)
    for i in range(steps):
        target = float(u[i, 0]) * cdf[-1]
        want = int(np.searchsorted(cdf, target, side="right"))
        assert hist[i] == want or abs(cdf[hist[i]] - target) < 1e-6 or abs(cdf[hist[i]] - probs[hist[i]] - target) < 1e-6, (i, hist[i], want)
    assert len(set(hist[:steps].tolist())) > 3  # different uniform numbers gave different tokens
