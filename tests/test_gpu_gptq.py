"""GPTQ on the device against the properties the reference's own test holds its numpy GPTQ to
(tests/python/test_gptq.py): with an identity Hessian it IS round-to-nearest, level for level; with a correlated
Hessian it is strictly better than round-to-nearest on ||X (W - W')^T||, moves the weights further, and is never
worse (x 1.02) on its own objective; plus the Hessian against numpy's 2 X^T X, and the column loop against a float64
numpy restatement of the published algorithm run here (most levels equal, output error within a few per cent)."""
import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


def correlated_inputs(rng, n, k, strength=0.9):
    base = rng.standard_normal((n, k))
    mix = np.eye(k) + strength * np.triu(np.ones((k, k)), 1) * rng.standard_normal((k, k)) / np.sqrt(k)
    return (base @ mix).astype(np.float32)


def output_error(x, w, wq):
    return float(np.linalg.norm(x @ (w - wq).T) / np.linalg.norm(x @ w.T))


def rtn(w, group=128):
    q, s, z = oracle.quantize_q4(w, group)
    return oracle.dequantize_q4(q, s, z, w.shape[1], group)


def gptq_numpy(w, hessian, group=128, percdamp=0.01):
    """The published algorithm in float64 numpy: column by column, parameters at each group's first column from the
    weights as they stand, error / U_jj pushed along row j of U."""
    from grilly2_b200.infer.gptq import inverse_cholesky
    upper, _ = inverse_cholesky(hessian, percdamp)
    work = w.astype(np.float64).copy()
    rows, k = w.shape
    levels = np.zeros((rows, k))
    deq = np.zeros((rows, k))
    for j in range(k):
        if j % group == 0:
            blk = work[:, j:j + group]
            lo, hi = blk.min(1), blk.max(1)
            scale = np.maximum((hi - lo) / 15, np.finfo(np.float32).eps)
        levels[:, j] = np.clip(np.round((work[:, j] - lo) / scale), 0, 15)
        deq[:, j] = levels[:, j] * scale + lo
        err = (work[:, j] - deq[:, j]) / upper[j, j]
        work[:, j + 1:] -= np.outer(err, upper[j, j + 1:])
    return levels, deq


def test_the_hessian_is_two_x_transpose_x_accumulated_over_calls():
    from grilly2_b200 import _C
    from grilly2_b200.infer.gptq import HessianAccumulator
    rng = np.random.default_rng(0)
    k = 200
    acc = HessianAccumulator(k)
    xs = [rng.standard_normal((n, k)).astype(np.float32) for n in (70, 1, 333)]
    for x in xs:
        acc.add(_C.Tensor.from_numpy(x))
    x = np.concatenate(xs).astype(np.float64)
    want = 2.0 * (x.T @ x)
    got = acc.hessian()
    assert acc.rows == 404 and np.array_equal(got, got.T)
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()


@pytest.mark.parametrize("group", [128, 64, 32])
def test_an_identity_hessian_is_round_to_nearest_exactly(group):
    from grilly2_b200.infer.gptq import gptq_quantize
    rng = np.random.default_rng(0)
    w = rng.standard_normal((37, 256)).astype(np.float32)
    q, s, z = oracle.quantize_q4(w, group)
    for mult in (1.0, 7.5):  # any multiple of I: the damping is relative
        t = gptq_quantize(w, mult * np.eye(256), group_size=group)
        np.testing.assert_array_equal(t._q.packed().numpy().view(np.uint32), q)
        np.testing.assert_array_equal(t._q.scale().numpy().view(np.uint32), s.view(np.uint32))
        np.testing.assert_array_equal(t._q.zero().numpy().view(np.uint32), z.view(np.uint32))


def test_it_beats_round_to_nearest_on_correlated_inputs_and_tracks_the_float64_algorithm():
    from grilly2_b200.infer.gptq import HessianAccumulator, gptq_quantize
    from grilly2_b200 import _C
    rng = np.random.default_rng(1)
    rows, k = 64, 512
    w = rng.standard_normal((rows, k)).astype(np.float32) * 0.1
    x = correlated_inputs(rng, 2048, k)
    acc = HessianAccumulator(k)
    acc.add(_C.Tensor.from_numpy(x))
    t = gptq_quantize(w, acc.hessian(), group_size=128)
    compensated = t.dequantize().numpy()
    plain = rtn(w)
    plain_error, gptq_error = output_error(x, w, plain), output_error(x, w, compensated)
    print(f"output error: rtn {plain_error:.4e}, gptq {gptq_error:.4e}, {plain_error / gptq_error:.2f}x")
    assert gptq_error < plain_error
    assert float(np.linalg.norm(w - compensated)) > float(np.linalg.norm(w - plain)), "GPTQ should move the weights further, not nearer"
    levels64, deq64 = gptq_numpy(w, 2.0 * (x.astype(np.float64).T @ x.astype(np.float64)))
    got_levels = oracle.unpack_q4(t._q.packed().numpy().view(np.uint32), k)
    same = float((got_levels == levels64).mean())
    ref_error = output_error(x, w, deq64.astype(np.float32))
    print(f"levels equal to the float64 loop: {same:.4f}; its output error {ref_error:.4e}")
    assert same >= 0.97 and gptq_error <= ref_error * 1.05


def test_it_is_never_worse_than_round_to_nearest_on_its_own_objective():
    from grilly2_b200.infer.gptq import gptq_quantize
    rng = np.random.default_rng(2)
    for trial in range(4):
        rows, k = 16, 256
        w = rng.standard_normal((rows, k)).astype(np.float32)
        x = correlated_inputs(rng, 1024, k, strength=0.3 * trial)
        hessian = 2.0 * (x.T @ x)
        plain = output_error(x, w, rtn(w))
        gptq = output_error(x, w, gptq_quantize(w, hessian, group_size=128).dequantize().numpy())
        assert gptq <= plain * 1.02, f"trial {trial}: {gptq:.3e} against {plain:.3e}"


def test_a_layer_sized_weight_and_the_refusals():
    """896 x 4864 (the down projection of the int8 full-step configuration): the loop runs 38 blocks; the quantized
    layer is loadable and its linear equals the linear of its dequantized weight."""
    import grilly2_b200 as g
    import grilly2_b200.nn.functional as F
    from grilly2_b200.infer.gptq import gptq_quantize
    rng = np.random.default_rng(3)
    n, k = 896, 4864
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    x = correlated_inputs(rng, 512, k, strength=0.5)
    hessian = 2.0 * (x.astype(np.float64).T @ x.astype(np.float64))
    t = gptq_quantize(w, hessian)
    deq = t.dequantize().numpy()
    assert output_error(x, w, deq) < output_error(x, w, rtn(w))
    xs = rng.standard_normal((2, k)).astype(np.float32)
    y = F.linear(g.from_numpy(xs), t).numpy()
    want = xs.astype(np.float64) @ deq.astype(np.float64).T
    assert np.abs(y - want).max() <= 1e-5 * np.abs(want).max()
    with pytest.raises(ValueError, match="whole number of groups"):
        gptq_quantize(w[:, :200], hessian[:200, :200])
    with pytest.raises(NotImplementedError, match="act_order"):
        gptq_quantize(w, hessian, act_order=True)
