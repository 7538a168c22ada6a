"""The frozen-weight backward of the quantized linear on the GPU, held to the reference's own test of it
(crates/grilly-infer/tests/quant.rs:14-17,168-216): against float64 over the DEQUANTIZED weight,
  |grad_x - want| <= (out_features + 2) * 2^-24 * sum|grad * w|,
  |grad_b - want| <= (rows + 2) * 2^-24 * sum|grad|,
and the Python test's rtol 1e-5 / atol 1e-6 against a float32 matrix product
(tests/python/test_quantization.py:111-126). The dequantized weight is the oracle's (bit-exact with the device's)."""
import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu

U = 2.0 ** -24

# (rows of grad, out_features, in_features): the reference's own case first, then ragged tiles, whole tiles, one row
SHAPES = [(5, 7, 37), (1, 1, 1), (3, 130, 70), (64, 64, 64), (65, 33, 129), (2, 300, 200), (1, 1152, 896), (130, 96, 260)]


def check(gx, gb, g, wd):
    g64, w64 = g.astype(np.float64), wd.astype(np.float64)
    want, mag = g64 @ w64, np.abs(g64) @ np.abs(w64)
    n = g.shape[1]
    assert (np.abs(gx.astype(np.float64) - want) <= (n + 2) * U * mag + np.finfo(np.float64).tiny).all()
    np.testing.assert_allclose(gx, (g @ wd).astype(np.float32), rtol=1e-5, atol=1e-6 * max(1.0, float(np.abs(want).max())))
    wantb, magb = g64.sum(axis=0), np.abs(g64).sum(axis=0)
    assert (np.abs(gb.astype(np.float64) - wantb) <= (g.shape[0] + 2) * U * magb + np.finfo(np.float64).tiny).all()


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_int8_backward_reaches_input_and_bias(m, n, k):
    from grilly2_b200 import _C
    w = oracle.xorshift_data(n * k, 11, -1.0, 1.0).reshape(n, k)
    g = oracle.xorshift_data(m * n, 14, -1.0, 1.0).reshape(m, n)
    q, scale = oracle.quantize_q8(w)
    wd = oracle.dequantize_q8(q, scale, k)
    weight = _C.Int8Weight.quantize(_C.Tensor.from_numpy(w))
    np.testing.assert_array_equal(weight.dequantize().numpy(), wd)
    gx, gb = weight.linear_backward(_C.Tensor.from_numpy(g), need_input=True, need_bias=True)
    assert gx.shape == (m, k) and gb.shape == (n,)
    check(gx.numpy(), gb.numpy(), g, wd)


@pytest.mark.parametrize("m,n,k", SHAPES)
@pytest.mark.parametrize("group", [32, 128])
def test_int4_backward_reaches_input_and_bias(m, n, k, group):
    from grilly2_b200 import _C
    w = oracle.xorshift_data(n * k, 11, -1.0, 1.0, int4_form=True).reshape(n, k)
    g = oracle.xorshift_data(m * n, 14, -1.0, 1.0, int4_form=True).reshape(m, n)
    q, scale, zero = oracle.quantize_q4(w, group)
    wd = oracle.dequantize_q4(q, scale, zero, k, group)
    weight = _C.Int4Weight.quantize(_C.Tensor.from_numpy(w), group)
    np.testing.assert_array_equal(weight.dequantize().numpy(), wd)
    gx, gb = weight.linear_backward(_C.Tensor.from_numpy(g), need_input=True, need_bias=True)
    check(gx.numpy(), gb.numpy(), g, wd)


def test_backward_keeps_leading_dimensions_and_skips_what_is_not_needed():
    from grilly2_b200 import _C
    n, k = 24, 40
    w = oracle.xorshift_data(n * k, 3, -1.0, 1.0).reshape(n, k)
    g = oracle.xorshift_data(2 * 3 * n, 4, -1.0, 1.0).reshape(2, 3, n)
    weight = _C.Int8Weight.quantize(_C.Tensor.from_numpy(w))
    gx, gb = weight.linear_backward(_C.Tensor.from_numpy(g))
    assert gx.shape == (2, 3, k) and gb is None
    wd = weight.dequantize().numpy()
    np.testing.assert_allclose(gx.numpy().reshape(6, k), g.reshape(6, n) @ wd, rtol=1e-5, atol=1e-5)
    gx, gb = weight.linear_backward(_C.Tensor.from_numpy(g), need_input=False, need_bias=True)
    assert gx is None
    np.testing.assert_allclose(gb.numpy(), g.reshape(6, n).sum(axis=0), rtol=1e-5, atol=1e-6)
    with pytest.raises(RuntimeError, match="out_features"):
        weight.linear_backward(_C.Tensor.from_numpy(np.zeros((2, n + 1), dtype=np.float32)))
