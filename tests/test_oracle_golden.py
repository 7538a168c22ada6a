"""The CPU oracle against the committed golden vectors and the reference
tests' known answers. No GPU. Bit-exact throughout: these are the pins that
let the oracle stand in for the reference (see tests/golden/make_golden.py
for where each fixture comes from)."""
import os

import numpy as np
import pytest

import oracle


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def cases(path):
    z = np.load(path)
    for i in range(int(z["count"])):
        yield i, z


def test_int8_matches_the_torch_formula_fixture(golden_dir):
    for i, z in cases(os.path.join(golden_dir, "int8_formula.npz")):
        w = z[f"w{i}"]
        q, scale = oracle.quantize_q8(w)
        k = w.shape[1]
        assert q.shape == (w.shape[0], oracle.words8(k))
        np.testing.assert_array_equal(oracle.unpack_q8(q, k), z[f"q{i}"], f"case {i} q")
        np.testing.assert_array_equal(bits(scale), bits(z[f"scale{i}"]), f"case {i} scale")
        np.testing.assert_array_equal(bits(oracle.dequantize_q8(q, scale, k)), bits(z[f"deq{i}"]), f"case {i} deq")
        # padding bytes of every row are zero (g2-quantize-q8.glsl:40-51)
        raw = q.view(np.uint8).reshape(w.shape[0], -1)
        assert not raw[:, k:].any()


def test_int8_known_answers():
    """crates/grilly-infer/tests/quant.rs:72-83: zero row -> scale eps, q 0;
    +-2.55 with amax 2.55 -> +127 / -128; 0.01 -> tie at 0.5 -> 0."""
    w = np.zeros((3, 5), dtype=np.float32)
    w[1] = [1, -1, 0.5, 0.25, 0]
    w[2, :3] = [2.55, -2.55, 0.01]
    q, scale = oracle.quantize_q8(w)
    v = oracle.unpack_q8(q, 5)
    assert scale[0] == np.float32(1.1920928955078125e-7) and not v[0].any()
    assert v[2, 0] == 127 and v[2, 1] == -128 and v[2, 2] == 0
    assert scale[2] == np.float32(2.55) / np.float32(127.5)


@pytest.mark.parametrize("name", ["int4_rtn.npz", "int4_formula.npz"])
def test_int4_matches_the_reference_fixtures(golden_dir, name):
    """int4_rtn.npz is the reference's own numpy rtn_quantize; int4_formula.npz
    the torch formula of its tests."""
    for i, z in cases(os.path.join(golden_dir, name)):
        w, group = z[f"w{i}"], int(z[f"group{i}"])
        k = w.shape[1]
        q, scale, zero = oracle.quantize_q4(w, group)
        np.testing.assert_array_equal(oracle.unpack_q4(q, k), z[f"levels{i}"], f"{name} case {i} levels")
        np.testing.assert_array_equal(bits(scale), bits(z[f"scale{i}"]), f"{name} case {i} scale")
        np.testing.assert_array_equal(bits(zero), bits(z[f"zero{i}"]), f"{name} case {i} zero")
        # packing == Int4Tensor.from_parts' host packer, padding words zero
        np.testing.assert_array_equal(q, oracle.pack_levels_q4(z[f"levels{i}"]))
        # dequantize is one fma per element (crates/grilly-infer/tests/quant4.rs:115-127)
        lv = z[f"levels{i}"].astype(np.float64)
        s = np.repeat(scale.astype(np.float64), group, axis=1)[:, :k]
        lo = np.repeat((zero - np.float32(8) * scale).astype(np.float64), group, axis=1)[:, :k]
        want = (lv * s + lo).astype(np.float32)  # exact product + one rounding == fma
        np.testing.assert_array_equal(bits(oracle.dequantize_q4(q, scale, zero, k, group)), bits(want))


def test_int4_ragged_group_and_nbytes():
    """k=130, group 128: the second group holds two values; rows pad to 20
    words (crates/grilly-infer/tests/quant4.rs:141-144 for the byte count)."""
    w = oracle.xorshift_data(5 * 130, 5 + 130 + 128, -1.5, 1.0, int4_form=True).reshape(5, 130)
    q, scale, zero = oracle.quantize_q4(w, 128)
    assert q.shape == (5, 20) and scale.shape == (5, 2)
    assert not (q[:, 17:] != 0).any() and not (q[:, 16] >> 8).any()
    n, k = 896, 4864
    assert n * (oracle.words4(k) * 4 + 8 * (-(-k // 128))) == n * ((-(-k // 32)) * 16 + 8 * (-(-k // 128)))


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (1, 5, 17), (3, 4, 16), (8, 7, 33), (9, 6, 100), (20, 13, 896),
                                   (1, 64, 4864), (16, 5, 33)])
@pytest.mark.parametrize("with_bias", [False, True])
def test_int8_linear_orders_are_within_the_reference_bound(m, n, k, with_bias):
    """Both summation orders against float64 under the bound of
    crates/grilly-infer/tests/quant.rs:136-160."""
    w = oracle.xorshift_data(n * k, m + n + k, -1.0, 1.0).reshape(n, k)
    x = oracle.xorshift_data(m * k, m * n * k + 7, -2.0, 2.0).reshape(m, k)
    b = oracle.xorshift_data(n, 99, -0.5, 0.5) if with_bias else None
    q, scale = oracle.quantize_q8(w)
    want, mag = oracle.linear_q8_f64(x, q, scale, b, k)
    tiny = np.finfo(np.float64).tiny
    for fn, terms in ((oracle.linear_q8, 16 * -(-(-(-k // 16)) // 64)), (oracle.linear_q8_tiled, k)):
        y = fn(x, q, scale, b, k)
        bound = (terms + 8) * 2.0 ** -24 * mag + tiny
        assert (np.abs(y - want) <= bound).all()


@pytest.mark.parametrize("m,n,k,group", [(1, 1, 32, 32), (1, 5, 128, 128), (3, 4, 130, 128), (8, 7, 256, 64),
                                         (2, 64, 896, 128), (9, 6, 4864, 128)])
@pytest.mark.parametrize("x_vec4", [False, True])
def test_int4_linear_is_within_the_reference_bound(m, n, k, group, x_vec4):
    """crates/grilly-infer/tests/quant4.rs:154-204."""
    if x_vec4 and k % 4:
        pytest.skip("the vec4 path needs k % 4 == 0")
    w = oracle.xorshift_data(n * k, m + n + k, -1.0, 1.0, int4_form=True).reshape(n, k)
    x = oracle.xorshift_data(m * k, m * n * k + 7, -2.0, 2.0, int4_form=True).reshape(m, k)
    b = oracle.xorshift_data(n, 99, -0.5, 0.5, int4_form=True)
    q, scale, zero = oracle.quantize_q4(w, group)
    for bias in (None, b):
        want, mag = oracle.linear_q4_f64(x, q, scale, zero, bias, k, group)
        y = oracle.linear_q4(x, q, scale, zero, bias, k, group, x_vec4)
        bound = (-(-k // 64) + 6 + 8) * 2.0 ** -24 * mag + np.finfo(np.float64).tiny
        assert (np.abs(y - want) <= bound).all()


def test_int4_linear_equals_linear_of_its_dequantized_weight():
    """tests/python/test_quantization.py:242-257."""
    rng = np.random.default_rng(3)
    rows, k, n = 3, 896, 64
    x = rng.standard_normal((rows, k)).astype(np.float32)
    w = (rng.standard_normal((n, k)) * 0.1).astype(np.float32)
    q, scale, zero = oracle.quantize_q4(w, 128)
    got = oracle.linear_q4(x, q, scale, zero, None, k, 128).astype(np.float64)
    deq = oracle.dequantize_q4(q, scale, zero, k, 128).astype(np.float64)
    want = x.astype(np.float64) @ deq.T
    magnitude = np.abs(x.astype(np.float64)) @ np.abs(deq).T
    assert (np.abs(got - want) / ((k // 64 + 14) * 2.0 ** -24 * magnitude)).max() <= 1.0


def test_cat_of_rows_is_exact():
    """Row concatenation is exact because parameters are per row / per
    (row, group) (crates/grilly-infer/src/quant.rs:171-223): quantizing a
    stacked weight equals stacking the quantized parts."""
    rng = np.random.default_rng(5)
    a, b = (rng.standard_normal((n, 200)).astype(np.float32) for n in (3, 6))
    qa, sa = oracle.quantize_q8(a)
    qb, sb = oracle.quantize_q8(b)
    qc, sc = oracle.quantize_q8(np.concatenate([a, b]))
    np.testing.assert_array_equal(np.concatenate([qa, qb]), qc)
    np.testing.assert_array_equal(bits(np.concatenate([sa, sb])), bits(sc))
