"""GPU parity of the dequant-fused linear: CUDA against the CPU oracle on the
same seeded inputs, through the C ABI.

Tolerances, written here as the tests state them:
 * GQ_KERNEL_GEMV (float32, the reference shader's summation order) against
   the oracle's float32 evaluation in that order: EQUAL;
 * GQ_KERNEL_DP4A (the fast path AUTO picks: exact integer dot products on
   fixed-point digit planes of x) against the same oracle:
   max|y - y_ref| / max|y_ref| <= 1e-5;
 * both against float64: the reference's own bound
   (crates/grilly-infer/tests/quant.rs:136-160, quant4.rs:170-196).
"""
import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu

TOL = 1e-5


@pytest.fixture(scope="module")
def g():
    import grilly2_b200 as g
    return g


def rel(y, ref):
    return float(np.abs(y - ref).max() / max(np.abs(ref).max(), np.finfo(np.float32).tiny))


INT8_SHAPES = [(1, 1, 1), (2, 300, 200), (1, 2500, 64), (2, 151, 4864), (1, 5, 17), (3, 4, 16), (8, 7, 33), (9, 6, 100), (20, 13, 896), (1, 64, 4864), (16, 5, 33),
               (2, 37, 1040), (4, 130, 2048), (1, 4864, 896), (5, 1152, 896)]


@pytest.mark.parametrize("m,n,k", INT8_SHAPES)
@pytest.mark.parametrize("with_bias", [False, True], ids=["nobias", "bias"])
def test_int8_linear(g, m, n, k, with_bias):
    from grilly2_b200 import _lib
    from grilly2_b200.infer.quantization import Int8Tensor
    w = oracle.xorshift_data(n * k, m + n + k, -1.0, 1.0).reshape(n, k)
    x = oracle.xorshift_data(m * k, m * n * k + 7, -2.0, 2.0).reshape(m, k)
    b = oracle.xorshift_data(n, 99, -0.5, 0.5) if with_bias else None
    t = Int8Tensor.from_hp(g.from_numpy(w))
    q, scale = oracle.quantize_q8(w)
    xt, bt = g.from_numpy(x)._t, None if b is None else g.from_numpy(b)._t
    ref = oracle.linear_q8(x, q, scale, b, k)
    want, mag = oracle.linear_q8_f64(x, q, scale, b, k)
    terms = 16 * -(-(-(-k // 16)) // 64)
    bound = (terms + 8) * 2.0 ** -24 * mag + np.finfo(np.float64).tiny
    y = t._q.linear(xt, bt, _lib.KERNEL_GEMV).numpy()
    np.testing.assert_array_equal(y, ref)  # same summation order as the reference's decode shader
    assert (np.abs(y - want) <= bound).all()
    kernels = [_lib.KERNEL_DP4A, _lib.KERNEL_AUTO, _lib.KERNEL_TENSOR_I8] + ([_lib.KERNEL_IMMA, _lib.KERNEL_UMMA] if m <= 2 else [])
    for kernel in kernels:
        y = t._q.linear(xt, bt, kernel).numpy()
        assert rel(y, ref) <= TOL
        assert (np.abs(y - want) <= bound).all()


INT4_SHAPES = [(1, 1, 32, 32), (2, 300, 384, 128), (1, 2500, 128, 128), (2, 151, 4864, 256), (1, 777, 1000, 128),
               (1, 5, 128, 128), (3, 4, 130, 128), (8, 7, 256, 64), (2, 64, 896, 128),
               (9, 6, 4864, 128), (4, 33, 4096, 128), (16, 40, 1024, 32), (1, 300, 8192, 128), (5, 7, 70, 32),
               (1, 2500, 512, 128), (1, 333, 4096, 128), (1, 97, 14336, 128), (2, 1500, 1024, 128), (2, 40, 12288, 128), (2, 700, 4096, 128), (3, 100, 4096, 128), (4, 333, 4096, 128), (16, 200, 4096, 128), (9, 50, 4096, 128), (8, 90, 8192, 128),
               (5, 33, 8192, 128), (1, 7, 4096, 128), (4, 1, 4096, 128), (1, 16, 8192, 128), (13, 17, 4096, 128),
               (1, 3000, 16384, 128)]


@pytest.mark.parametrize("m,n,k,group", INT4_SHAPES)
@pytest.mark.parametrize("with_bias", [False, True], ids=["nobias", "bias"])
def test_int4_linear(g, m, n, k, group, with_bias):
    from grilly2_b200 import _lib
    from grilly2_b200.infer.quantization import Int4Tensor
    w = oracle.xorshift_data(n * k, m + n + k, -1.0, 1.0, int4_form=True).reshape(n, k)
    x = oracle.xorshift_data(m * k, m * n * k + 7, -2.0, 2.0, int4_form=True).reshape(m, k)
    b = oracle.xorshift_data(n, 99, -0.5, 0.5, int4_form=True) if with_bias else None
    t = Int4Tensor.from_hp(g.from_numpy(w), group)
    q, scale, zero = oracle.quantize_q4(w, group)
    xt, bt = g.from_numpy(x)._t, None if b is None else g.from_numpy(b)._t
    ref = oracle.linear_q4(x, q, scale, zero, b, k, group)  # x at offset 0: vec4 iff k % 4 == 0
    want, mag = oracle.linear_q4_f64(x, q, scale, zero, b, k, group)
    bound = (-(-k // 64) + 14) * 2.0 ** -24 * mag + np.finfo(np.float64).tiny
    y = t._q.linear(xt, bt, _lib.KERNEL_GEMV).numpy()
    np.testing.assert_array_equal(y, ref)
    assert (np.abs(y - want) <= bound).all()
    kernels = [_lib.KERNEL_DP4A, _lib.KERNEL_AUTO] + ([_lib.KERNEL_IMMA] if m <= 2 and group % 128 == 0 else [])
    kernels += [_lib.KERNEL_RING] if group == 128 and m <= 16 and k in (4096, 8192) else []
    kernels += [_lib.KERNEL_UMMA] if group == 128 and m <= 16 and k % 128 == 0 else []  # tcgen05: one pass for up to 16 rows
    kernels += [_lib.KERNEL_UMMA_LANES] if group == 128 and m <= 16 and k % 128 == 0 and k <= 16384 else []  # the same with the features on the lanes
    for kernel in kernels:
        y = t._q.linear(xt, bt, kernel).numpy()
        assert rel(y, ref) <= TOL
        assert (np.abs(y - want) <= bound).all()


def test_int4_many_rows_go_in_passes_of_sixteen(g):
    """More than 16 rows of x through a large int4 group-128 layer: AUTO runs the tcgen05 kernel in passes of 16 rows,
    so the result equals that kernel's on each block of rows bit for bit, and the oracle within the decode tolerance."""
    from grilly2_b200 import _C, _lib
    m, n, k = 40, 2100, 4096
    rng = np.random.default_rng(40)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal(n).astype(np.float32)
    w4 = _C.Int4Weight.quantize(_C.Tensor.from_numpy(w), 128)
    q4, s4, z4 = oracle.quantize_q4(w, 128)
    y = w4.linear(_C.Tensor.from_numpy(x), _C.Tensor.from_numpy(b)).numpy()
    assert rel(y, oracle.linear_q4_f64(x, q4, s4, z4, b, k, 128)[0]) <= TOL
    for r in range(0, m, 16):
        part = w4.linear(_C.Tensor.from_numpy(x[r:r + 16]), _C.Tensor.from_numpy(b), _lib.KERNEL_UMMA_LANES).numpy()
        np.testing.assert_array_equal(y[r:r + 16], part)


@pytest.mark.parametrize("x_off", [1, 2, 4])
def test_x_and_bias_at_element_offsets(g, x_off):
    """x may start at any element (crates/grilly-core/src/kernel.rs:26-36);
    off a multiple of four the scalar path runs, whose int4 `sum` order is the
    reference's scalar one (g2-linear-q4.glsl:80-86)."""
    from grilly2_b200 import _C, _lib
    rng = np.random.default_rng(x_off)
    m, n, k = 3, 21, 4096
    w = rng.standard_normal((n, k)).astype(np.float32)
    flat = rng.standard_normal(x_off + m * k).astype(np.float32)
    bflat = rng.standard_normal(5 + n).astype(np.float32)
    xs = _C.Tensor(_C.Tensor.from_numpy(flat).storage, (m, k), "float32", x_off)
    bs = _C.Tensor(_C.Tensor.from_numpy(bflat).storage, (n,), "float32", 5)
    x, b = flat[x_off:].reshape(m, k), bflat[5:]
    w8 = _C.Int8Weight.quantize(_C.Tensor.from_numpy(w))
    q, scale = oracle.quantize_q8(w)
    ref8 = oracle.linear_q8(x, q, scale, b, k)
    np.testing.assert_array_equal(w8.linear(xs, bs, _lib.KERNEL_GEMV).numpy(), ref8)
    assert rel(w8.linear(xs, bs, _lib.KERNEL_DP4A).numpy(), ref8) <= TOL
    assert rel(w8.linear(_C.Tensor(xs.storage, (1, k), "float32", x_off), bs, _lib.KERNEL_IMMA).numpy(), ref8[:1]) <= TOL
    assert rel(w8.linear(xs, bs, _lib.KERNEL_TENSOR_I8).numpy(), ref8) <= TOL  # its digit-plane kernel reads x element by element there
    w4 = _C.Int4Weight.quantize(_C.Tensor.from_numpy(w), 64)
    q4, s4, z4 = oracle.quantize_q4(w, 64)
    ref = oracle.linear_q4(x, q4, s4, z4, b, k, 64, x_vec4=(x_off % 4 == 0))
    np.testing.assert_array_equal(w4.linear(xs, bs, _lib.KERNEL_GEMV).numpy(), ref)
    assert rel(w4.linear(xs, bs, _lib.KERNEL_DP4A).numpy(), ref) <= TOL
    w4g = _C.Int4Weight.quantize(_C.Tensor.from_numpy(w), 128)
    q4, s4, z4 = oracle.quantize_q4(w, 128)
    ref = oracle.linear_q4(x[:1], q4, s4, z4, b, k, 128, x_vec4=(x_off % 4 == 0))
    assert rel(w4g.linear(_C.Tensor(xs.storage, (1, k), "float32", x_off), bs, _lib.KERNEL_RING).numpy(), ref) <= TOL
    ref3 = oracle.linear_q4_f64(x, q4, s4, z4, b, k, 128)[0]
    for kernel in (_lib.KERNEL_UMMA_LANES, _lib.KERNEL_UMMA):  # the tcgen05 kernels fetch x sixteen bytes at a time
        if x_off % 4 == 0:
            assert rel(w4g.linear(xs, bs, kernel).numpy(), ref3) <= TOL
        else:
            with pytest.raises(RuntimeError, match="16-byte aligned x"):
                w4g.linear(xs, bs, kernel)
    assert rel(w4g.linear(xs, bs).numpy(), ref3) <= TOL  # AUTO answers either way


def test_leading_dims_empty_and_refusals(g):
    """crates/grilly-infer/tests/quant.rs:220-253."""
    from grilly2_b200.infer.quantization import Int4Tensor, Int8Tensor
    import grilly2_b200.nn.functional as F
    rng = np.random.default_rng(6)
    n, k = 6, 64
    w = rng.standard_normal((n, k)).astype(np.float32)
    x = rng.standard_normal((2, 3, k)).astype(np.float32)
    for t in (Int8Tensor.from_hp(g.from_numpy(w)), Int4Tensor.from_hp(g.from_numpy(w), 32)):
        flat = F.linear(g.from_numpy(x.reshape(6, k)), t)
        batched = F.linear(g.from_numpy(x), t)
        assert tuple(batched.shape) == (2, 3, n)
        np.testing.assert_array_equal(batched.numpy().reshape(6, n), flat.numpy())
        assert tuple(F.linear(g.from_numpy(np.zeros((0, k), dtype=np.float32)), t).shape) == (0, n)
        with pytest.raises(RuntimeError, match="does not end in in_features"):
            F.linear(g.from_numpy(np.zeros((2, 7), dtype=np.float32)), t)
        with pytest.raises(RuntimeError, match="bias must be"):
            F.linear(g.from_numpy(x), t, g.from_numpy(np.zeros(n + 1, dtype=np.float32)))


def test_cat_linear_equals_separate_linears(g):
    """A fused q/k/v projection computes each row exactly as the separate
    ones did (crates/grilly-infer/tests/fused_ops.rs:194-228)."""
    from grilly2_b200.infer.quantization import Int4Tensor, Int8Tensor
    import grilly2_b200.nn.functional as F
    rng = np.random.default_rng(8)
    parts = [rng.standard_normal((n, 896)).astype(np.float32) * 0.02 for n in (896, 128, 128)]
    x = g.from_numpy(rng.standard_normal((1, 896)).astype(np.float32))
    for cls, extra in ((Int8Tensor, ()), (Int4Tensor, (128,))):
        qs = [cls.from_hp(g.from_numpy(p), *extra) for p in parts]
        fused = F.linear(x, cls._cat(qs)).numpy()
        separate = np.concatenate([F.linear(x, q).numpy() for q in qs], axis=1)
        np.testing.assert_array_equal(fused, separate)


@pytest.mark.parametrize("config", ["c1", "c2", "c3"])
def test_benchmark_configs_full_size(g, config):
    """The benchmark's own shapes and seeds. The oracle finishes these in
    seconds, so the comparison is outright; linearity in x is checked on top
    as a size-independent property."""
    from grilly2_b200 import _lib
    from grilly2_b200.infer.quantization import Int4Tensor, Int8Tensor
    import grilly2_b200.nn.functional as F
    if config == "c1":
        rng = np.random.default_rng(0)
        x = rng.standard_normal((1, 896)).astype(np.float32)
        w = (rng.standard_normal((4864, 896)) * 0.02).astype(np.float32)
        t = Int8Tensor.from_hp(g.from_numpy(w))
        q, scale = oracle.quantize_q8(w)
        ref = oracle.linear_q8(x, q, scale, None, 896)
        ms = [1]
    else:
        n, k, sigma, seed, ms = (14336, 4096, 0.02, 1, [1, 4, 16]) if config == "c2" else (28672, 8192, 0.015, 2, [1, 8, 16])
        rng = np.random.default_rng(seed)
        x = rng.standard_normal((max(ms), k)).astype(np.float32)
        w = (rng.standard_normal((n, k)) * sigma).astype(np.float32)
        t = Int4Tensor.from_hp(g.from_numpy(w), 128)
        q, scale, zero = oracle.quantize_q4(w, 128)
        np.testing.assert_array_equal(t._q.packed().numpy().view(np.uint32), q)
    for m in ms:
        xm = x[:m]
        if config != "c1":
            ref = oracle.linear_q4(xm, q, scale, zero, None, xm.shape[1], 128)
        y = F.linear(g.from_numpy(xm), t).numpy()  # AUTO: the fast path
        assert rel(y, ref) <= TOL
        np.testing.assert_array_equal(t._q.linear(g.from_numpy(xm)._t, None, _lib.KERNEL_GEMV).numpy(), ref)
    # linearity: f(2x) == 2 f(x) exactly (scaling by two is exact in binary floating point)
    y1 = F.linear(g.from_numpy(x[:1]), t).numpy()
    y2 = F.linear(g.from_numpy(2 * x[:1]), t).numpy()
    np.testing.assert_array_equal(y2, 2 * y1)


def test_dp4a_digit_planes_on_hard_inputs(g):
    """The fixed-point copy of x must stay exact enough where float ranges are
    wide: per-vector outliers (1e4 x the rest), tiny and huge magnitudes,
    exact zeros, negative zero. Non-finite x makes the affected outputs NaN."""
    from grilly2_b200 import _C, _lib
    rng = np.random.default_rng(12)
    n, k = 50, 4096
    w = rng.standard_normal((n, k)).astype(np.float32)
    x = rng.standard_normal((4, k)).astype(np.float32)
    x[0, ::97] *= 1e4
    x[1] *= 1e-30
    x[2] *= 1e30
    x[3, :512] = 0.0
    x[3, 600] = -0.0
    w8 = _C.Int8Weight.quantize(_C.Tensor.from_numpy(w))
    w4 = _C.Int4Weight.quantize(_C.Tensor.from_numpy(w), 128)
    q, scale = oracle.quantize_q8(w)
    q4, s4, z4 = oracle.quantize_q4(w, 128)
    for r in range(4):
        xr = x[r:r + 1]
        xt = _C.Tensor.from_numpy(xr)
        for kernel in (_lib.KERNEL_DP4A, _lib.KERNEL_IMMA):
            assert rel(w8.linear(xt, None, kernel).numpy(), oracle.linear_q8_f64(xr, q, scale, None, k)[0]) <= TOL
            assert rel(w4.linear(xt, None, kernel).numpy(), oracle.linear_q4_f64(xr, q4, s4, z4, None, k, 128)[0]) <= TOL
        assert rel(w4.linear(xt, None, _lib.KERNEL_RING).numpy(), oracle.linear_q4_f64(xr, q4, s4, z4, None, k, 128)[0]) <= TOL
        for kernel in (_lib.KERNEL_UMMA, _lib.KERNEL_UMMA_LANES):
            assert rel(w4.linear(xt, None, kernel).numpy(), oracle.linear_q4_f64(xr, q4, s4, z4, None, k, 128)[0]) <= TOL
    for kernel in (_lib.KERNEL_UMMA, _lib.KERNEL_UMMA_LANES):
        assert rel(w4.linear(_C.Tensor.from_numpy(x), None, kernel).numpy(), oracle.linear_q4_f64(x, q4, s4, z4, None, k, 128)[0]) <= TOL
    xbad = x[:1].copy()
    xbad[0, 5] = np.inf
    for kernel in (_lib.KERNEL_DP4A, _lib.KERNEL_IMMA):
        xbad[0, 5] = np.inf
        assert np.isnan(w8.linear(_C.Tensor.from_numpy(xbad), None, kernel).numpy()).all()
        xbad[0, 5] = np.nan
        assert np.isnan(w4.linear(_C.Tensor.from_numpy(xbad), None, kernel).numpy()).all()
    for bad in (np.inf, np.nan):
        xbad[0, 5] = bad
        assert np.isnan(w4.linear(_C.Tensor.from_numpy(xbad), None, _lib.KERNEL_RING).numpy()).all()
        assert np.isnan(w4.linear(_C.Tensor.from_numpy(xbad), None, _lib.KERNEL_UMMA).numpy()).all()
        assert np.isnan(w4.linear(_C.Tensor.from_numpy(xbad), None, _lib.KERNEL_UMMA_LANES).numpy()).all()


def test_outputs_that_overlap_inputs_are_refused(g):
    """Many CTAs read x while others already write y (and, in the fused norm, h_out): an output that shares memory with
    an input is reported, not computed."""
    import ctypes
    from grilly2_b200 import _C, _lib
    lib, ctx = _lib.load(), _C.context()
    rng = np.random.default_rng(2)
    k = n = 64
    w = rng.standard_normal((n, k)).astype(np.float32)
    w8 = _C.Int8Weight.quantize(_C.Tensor.from_numpy(w))
    w4 = _C.Int4Weight.quantize(_C.Tensor.from_numpy(w), 32)
    x = _C.Tensor.from_numpy(rng.standard_normal((1, k)).astype(np.float32))
    res = _C.Tensor.from_numpy(rng.standard_normal((1, k)).astype(np.float32))
    nw = _C.Tensor.from_numpy(np.ones(k, dtype=np.float32))
    y = _C.Tensor.empty((1, n), "float32")
    hx, hq, hs = x.storage.handle, w8._qt.storage.handle, w8._scale.storage.handle
    assert lib.gq_int8_linear(ctx, hx, 0, 1, k, hq, hs, 0, 0, n, hx, 0) == _lib.GQ_ERR and "overlap" in _lib.last_error()
    assert lib.gq_int4_linear(ctx, hx, 0, 1, k, w4._qt.storage.handle, w4._scale.storage.handle, w4._zero.storage.handle, 0, 0, n, 32, hx, 0) == _lib.GQ_ERR
    assert "overlap" in _lib.last_error()
    for h_out in (hx, res.storage.handle):  # the residual stream updated in place
        rc = lib.gq_int8_linear_norm(ctx, hx, res.storage.handle, nw.storage.handle, 1e-6, h_out, k, hq, hs, 0, 0, n, y.storage.handle)
        assert rc == _lib.GQ_ERR and "h_out must not overlap" in _lib.last_error()
    rc = lib.gq_int8_linear_norm(ctx, hx, res.storage.handle, nw.storage.handle, 1e-6, 0, k, hq, hs, 0, 0, n, hx)
    assert rc == _lib.GQ_ERR and "output must not overlap" in _lib.last_error()
    # a separate h_out is fine
    h = _C.Tensor.empty((1, k), "float32")
    _lib.check(lib.gq_int8_linear_norm(ctx, hx, res.storage.handle, nw.storage.handle, 1e-6, h.storage.handle, k, hq, hs, 0, 0, n, y.storage.handle))
    np.testing.assert_array_equal(h.numpy(), x.numpy() + res.numpy())
