"""GPU parity of the tensor-core prefill GEMMs (int8 weights) against the CPU oracle, through the C ABI.

Two kernels. GQ_KERNEL_TENSOR_I8 (what AUTO runs from 64 rows of x on): exact integer arithmetic against three
digit planes of a per-row fixed-point x; bound here: max|y - y_ref| / max|y_ref| <= 1e-5 against the oracle's
float64 value (the decode tolerance; x is held to 2^-23 of its row's largest value). GQ_KERNEL_TENSOR (tf32):
<= 2e-3, the tolerance the prefill configuration states, against the oracle's float32 evaluation in the
reference's tiled-kernel order (crates/grilly-core/shaders/g2-linear-q8-tiled.glsl:78-96); the int8 codes are
exact in tf32, only x is rounded.
"""
import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu

TOL = 2e-3      # tf32 kernel; the configuration's bound
TOL_I8 = 1e-5   # integer kernel


@pytest.fixture(scope="module")
def g():
    import grilly2_b200 as g
    return g


def rel(y, ref):
    return float(np.abs(y - ref).max() / max(np.abs(ref).max(), np.finfo(np.float32).tiny))


@pytest.mark.parametrize("m,n,k", [(64, 64, 128), (65, 130, 100), (128, 64, 4864), (256, 300, 512), (300, 1000, 896),
                                   (1, 128, 32), (513, 129, 36), (64, 4864, 896)])
@pytest.mark.parametrize("with_bias", [False, True], ids=["nobias", "bias"])
def test_prefill_matches_the_oracle(g, m, n, k, with_bias):
    from grilly2_b200 import _lib
    from grilly2_b200.infer.quantization import Int8Tensor
    rng = np.random.default_rng(m * 131 + n * 17 + k)
    w = rng.standard_normal((n, k)).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal(n).astype(np.float32) if with_bias else None
    t = Int8Tensor.from_hp(g.from_numpy(w))
    q, scale = oracle.quantize_q8(w)
    ref = oracle.linear_q8_tiled(x, q, scale, b, k)
    y = t._q.linear(g.from_numpy(x)._t, None if b is None else g.from_numpy(b)._t, _lib.KERNEL_TENSOR).numpy()
    assert rel(y, ref) <= TOL


@pytest.mark.parametrize("m,n,k", [(64, 64, 128), (65, 130, 100), (128, 64, 4864), (256, 300, 512), (300, 1000, 896), (1, 128, 32),
                                   (513, 129, 36), (64, 4864, 896), (5, 17, 37), (81, 257, 130), (160, 512, 4096), (79, 255, 127)])
@pytest.mark.parametrize("with_bias", [False, True], ids=["nobias", "bias"])
def test_integer_prefill_matches_the_oracle(g, m, n, k, with_bias):
    from grilly2_b200 import _lib
    from grilly2_b200.infer.quantization import Int8Tensor
    rng = np.random.default_rng(m * 131 + n * 17 + k)
    w = rng.standard_normal((n, k)).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal(n).astype(np.float32) if with_bias else None
    t = Int8Tensor.from_hp(g.from_numpy(w))
    q, scale = oracle.quantize_q8(w)
    ref = oracle.linear_q8_f64(x, q, scale, b, k)[0]
    bt = None if b is None else g.from_numpy(b)._t
    y = t._q.linear(g.from_numpy(x)._t, bt, _lib.KERNEL_TENSOR_I8).numpy()
    assert y.shape == (m, n) and rel(y, ref) <= TOL_I8
    if m >= 4:  # AUTO takes this kernel from three rows on (at three rows on weights of 8 MB and more)
        np.testing.assert_array_equal(t._q.linear(g.from_numpy(x)._t, bt).numpy(), y)


def test_integer_prefill_rows_are_independent_zero_rows_give_the_bias_and_bad_rows_give_nan(g):
    from grilly2_b200 import _lib
    from grilly2_b200.infer.quantization import Int8Tensor
    rng = np.random.default_rng(11)
    m, n, k = 100, 300, 260
    w = rng.standard_normal((n, k)).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal(n).astype(np.float32)
    t = Int8Tensor.from_hp(g.from_numpy(w))
    q, scale = oracle.quantize_q8(w)
    clean = t._q.linear(g.from_numpy(x)._t, g.from_numpy(b)._t, _lib.KERNEL_TENSOR_I8).numpy()
    x2 = x.copy()
    x2[3] = 0.0                      # a row of zeros: exactly the bias
    x2[7, 5] = np.inf                # non-finite rows: NaN outputs, the rows around them untouched
    x2[90, 259] = np.nan
    x2[50] *= 1e30                   # a large row and a tiny row keep their own exponents
    x2[51] *= 1e-25
    x2[60, 17] = 1000.0              # one outlier costs its own row precision (2^-23 of 1000 per element), no other row
    y = t._q.linear(g.from_numpy(x2)._t, g.from_numpy(b)._t, _lib.KERNEL_TENSOR_I8).numpy()
    np.testing.assert_array_equal(y[3], b)
    assert np.isnan(y[7]).all() and np.isnan(y[90]).all()
    touched = [3, 7, 90, 50, 51, 60]
    keep = np.setdiff1d(np.arange(m), touched)
    np.testing.assert_array_equal(y[keep], clean[keep])
    for r in (50, 51, 60):
        ref = oracle.linear_q8_f64(x2[r:r + 1], q, scale, b, k)[0]
        assert rel(y[r:r + 1], ref) <= TOL_I8


def test_integer_prefill_refuses_what_its_sums_cannot_hold(g):
    from grilly2_b200 import _C, _lib
    k = 131072 + 16
    wt = _C.Int8Weight.quantize(_C.Tensor.from_numpy(np.ones((1, k), dtype=np.float32)))
    x = _C.Tensor.from_numpy(np.ones((2, k), dtype=np.float32))
    with pytest.raises(RuntimeError, match="in_features up to 131072"):
        wt.linear(x, None, _lib.KERNEL_TENSOR_I8)
    with pytest.raises(RuntimeError, match="unknown kernel selector"):
        wt.linear(x, None, 8)


def test_prefill_refuses_shapes_it_cannot_map(g):
    from grilly2_b200 import _lib
    from grilly2_b200.infer.quantization import Int8Tensor
    rng = np.random.default_rng(0)
    w = rng.standard_normal((8, 33)).astype(np.float32)
    t = Int8Tensor.from_hp(g.from_numpy(w))
    x = g.from_numpy(rng.standard_normal((70, 33)).astype(np.float32))
    with pytest.raises(RuntimeError, match="in_features % 4 == 0"):
        t._q.linear(x._t, None, _lib.KERNEL_TENSOR)
    # AUTO answers with the integer kernel, which takes any in_features
    ref = oracle.linear_q8_f64(x.numpy(), *oracle.quantize_q8(w), None, 33)[0]
    assert rel(t._q.linear(x._t, None).numpy(), ref) <= TOL_I8


@pytest.mark.parametrize("m", [256, 2048, 8192])
def test_prefill_benchmark_shape(g, m):
    """Config 4: x [m, 4096], W [14336, 4096]. m = 256 is compared outright; at
    m = 2048 and m = 8192 a sample of rows is (rows of x are independent), plus the
    call-twice-equal property."""
    from grilly2_b200 import _lib
    from grilly2_b200.infer.quantization import Int8Tensor
    rng = np.random.default_rng(3)
    x = rng.standard_normal((m, 4096)).astype(np.float32)
    w = (rng.standard_normal((14336, 4096)) * 0.02).astype(np.float32)
    t = Int8Tensor.from_hp(g.from_numpy(w))
    q, scale = oracle.quantize_q8(w)
    y = t._q.linear(g.from_numpy(x)._t, None).numpy()
    rows = np.arange(m) if m <= 256 else rng.choice(m, 64, replace=False)
    ref = oracle.linear_q8_f64(x[rows], q, scale, None, 4096)[0]
    assert rel(y[rows], ref) <= TOL_I8  # (the configuration asks for 2e-3)
    y32 = t._q.linear(g.from_numpy(x)._t, None, _lib.KERNEL_TENSOR).numpy()  # the tf32 kernel on the same shape
    assert rel(y32[rows], oracle.linear_q8_tiled(x[rows], q, scale, None, 4096)) <= TOL
    np.testing.assert_array_equal(t._q.linear(g.from_numpy(x)._t, None).numpy(), y)  # deterministic
