"""GPU parity of the tensor-core prefill GEMM (int8 weights, tf32 MMA) against
the CPU oracle, through the C ABI.

Tolerance: max|y - y_ref| / max|y_ref| <= 2e-3 against the oracle's float32
evaluation in the reference's tiled-kernel order
(crates/grilly-core/shaders/g2-linear-q8-tiled.glsl:78-96); the int8 codes are
exact in tf32, only x is rounded.
"""
import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu

TOL = 2e-3


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
    if m >= 64:  # AUTO takes the same kernel from 64 rows on
        np.testing.assert_array_equal(t._q.linear(g.from_numpy(x)._t, None if b is None else g.from_numpy(b)._t).numpy(), y)


def test_prefill_refuses_shapes_it_cannot_map(g):
    from grilly2_b200 import _lib
    from grilly2_b200.infer.quantization import Int8Tensor
    rng = np.random.default_rng(0)
    t = Int8Tensor.from_hp(g.from_numpy(rng.standard_normal((8, 33)).astype(np.float32)))
    x = g.from_numpy(rng.standard_normal((70, 33)).astype(np.float32))
    with pytest.raises(RuntimeError, match="in_features % 4 == 0"):
        t._q.linear(x._t, None, _lib.KERNEL_TENSOR)
    # AUTO falls back to a GEMV and still answers
    ref = oracle.linear_q8(x.numpy(), *oracle.quantize_q8(t.dequantize().numpy() * 0 + rng.standard_normal((8, 33)).astype(np.float32)), None, 33)
    assert t._q.linear(x._t, None).numpy().shape == ref.shape


@pytest.mark.parametrize("m", [256, 2048, 8192])
def test_prefill_benchmark_shape(g, m):
    """Config 4: x [m, 4096], W [14336, 4096]. m = 256 is compared outright; at
    m = 2048 and m = 8192 a sample of rows is (rows of x are independent), plus the
    replay-equals-eager property."""
    from grilly2_b200.infer.quantization import Int8Tensor
    rng = np.random.default_rng(3)
    x = rng.standard_normal((m, 4096)).astype(np.float32)
    w = (rng.standard_normal((14336, 4096)) * 0.02).astype(np.float32)
    t = Int8Tensor.from_hp(g.from_numpy(w))
    q, scale = oracle.quantize_q8(w)
    y = t._q.linear(g.from_numpy(x)._t, None).numpy()
    rows = np.arange(m) if m <= 256 else rng.choice(m, 64, replace=False)
    ref = oracle.linear_q8_tiled(x[rows], q, scale, None, 4096)
    assert rel(y[rows], ref) <= TOL
    np.testing.assert_array_equal(t._q.linear(g.from_numpy(x)._t, None).numpy(), y)  # deterministic
