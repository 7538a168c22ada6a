"""The decode-step operators one by one, through the C ABI, against float64 numpy."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _env():
    from grilly2_b200 import _C, _lib
    return _C, _lib, _lib.load(), _C.context()


@pytest.mark.parametrize("rows,n", [(1, 151936), (3, 1000), (70, 257), (1, 1)])
def test_argmax_rows_first_maximum_wins(rows, n):
    _C, _lib, lib, ctx = _env()
    rng = np.random.default_rng(rows * 1000 + n)
    v = rng.standard_normal((rows, n)).astype(np.float32)
    if n > 10:
        v[0, 7] = v[0, n - 2] = 50.0           # a tie: the first index wins
        v[-1, :] = -np.abs(v[-1, :]) - 1.0     # an all-negative row
        v[-1, 3] = np.nan                      # NaN ranks below every number
    want = np.array([int(np.nanargmax(r)) for r in v], dtype=np.int32)
    t, out = _C.Tensor.from_numpy(v), _C.Tensor.empty((rows,), "int32")
    for _ in range(2):  # the state must return to zero between calls
        _lib.check(lib.gq_argmax_rows(ctx, t.storage.handle, rows, n, out.storage.handle))
        np.testing.assert_array_equal(out.numpy(), want)


@pytest.mark.parametrize("dim,heads,kv_heads,max_len,length", [(64, 14, 2, 1024, 1023), (64, 14, 2, 1024, 0), (32, 4, 2, 48, 20),
                                                               (128, 8, 8, 300, 299), (64, 2, 1, 40000, 33333)])
def test_attention_against_float64(dim, heads, kv_heads, max_len, length):
    """`length` positions are cached and the cursor says so; the kernel attends over length + 1 (the appended one)."""
    _C, _lib, lib, ctx = _env()
    rng = np.random.default_rng(dim + length)
    k = rng.standard_normal((kv_heads, max_len, dim)).astype(np.float32)
    v = rng.standard_normal((kv_heads, max_len, dim)).astype(np.float32)
    q = rng.standard_normal((heads, dim)).astype(np.float32)
    layers, layer = 3, 1
    lens = np.array([5, length, 9], dtype=np.int32)
    nbytes = ctypes.c_uint64()
    _lib.check(lib.gq_attn_scratch_bytes(ctx, heads, dim, max_len, ctypes.byref(nbytes)))
    scratch = _C.Tensor.from_numpy(np.zeros(nbytes.value // 4, dtype=np.float32))
    tq, tk, tv, tl = (_C.Tensor.from_numpy(a) for a in (q, k.reshape(-1), v.reshape(-1), lens))
    out = _C.Tensor.empty((heads, dim), "float32")
    n = min(length + 1, max_len)
    want = np.zeros((heads, dim))
    for h in range(heads):
        g = h // (heads // kv_heads)
        s = k[g, :n].astype(np.float64) @ q[h].astype(np.float64) / np.sqrt(dim)
        e = np.exp(s - s.max())
        want[h] = (e / e.sum()) @ v[g, :n].astype(np.float64)
    for _ in range(2):  # the counters in scratch reset themselves
        _lib.check(lib.gq_attn_decode(ctx, tq.storage.handle, tk.storage.handle, 0, tv.storage.handle, 0, tl.storage.handle, layer,
                                      layers, heads, kv_heads, dim, max_len, float(dim) ** -0.5, scratch.storage.handle,
                                      out.storage.handle))
        got = out.numpy()
        assert np.abs(got - want).max() <= 2e-6 * max(1.0, np.abs(want).max())


def test_attention_refuses_other_head_sizes():
    _C, _lib, lib, ctx = _env()
    t = _C.Tensor.from_numpy(np.zeros(4096, dtype=np.float32))
    ti = _C.Tensor.from_numpy(np.zeros(1, dtype=np.int32))
    rc = lib.gq_attn_decode(ctx, t.storage.handle, t.storage.handle, 0, t.storage.handle, 0, ti.storage.handle, 0, 1, 2, 1, 48, 8,
                            1.0, t.storage.handle, t.storage.handle)
    assert rc != 0 and b"head_dim" in lib.gq_last_error()


@pytest.mark.parametrize("k,n", [(896, 1152), (4864, 896), (896, 151936), (64, 5)])
def test_fused_norm_and_swiglu_linears_equal_the_separate_operators(k, n):
    """gq_int8_linear_norm == gq_add_rms_norm then gq_int8_linear; gq_int8_linear_swiglu == gq_swiglu then gq_int8_linear (to 2e-6)."""
    _C, _lib, lib, ctx = _env()
    rng = np.random.default_rng(k + n)
    w = _C.Int8Weight.quantize(_C.Tensor.from_numpy((rng.standard_normal((n, k)) * 0.05).astype(np.float32)))
    x, res = (_C.Tensor.from_numpy(rng.standard_normal((1, k)).astype(np.float32)) for _ in range(2))
    nw = _C.Tensor.from_numpy((1 + 0.1 * rng.standard_normal(k)).astype(np.float32))
    bias = _C.Tensor.from_numpy(rng.standard_normal(n).astype(np.float32))
    for residual in (res, None):
        xn, h = _C.Tensor.empty((1, k), "float32"), _C.Tensor.empty((1, k), "float32")
        _lib.check(lib.gq_add_rms_norm(ctx, x.storage.handle, residual.storage.handle if residual is not None else 0, nw.storage.handle, 1, k,
                                       1e-6, xn.storage.handle, h.storage.handle))
        want = w.linear(xn, bias, _lib.KERNEL_IMMA).numpy()
        got, hs = w.linear_norm(x, residual, nw, 1e-6, bias, True)
        np.testing.assert_array_equal(hs.numpy(), h.numpy())
        assert np.abs(got.numpy() - want).max() <= 1e-6 * np.abs(want).max()
        got2, none = w.linear_norm(x, residual, nw, 1e-6, bias, False)
        assert none is None
        np.testing.assert_array_equal(got2.numpy(), got.numpy())
    gu = _C.Tensor.from_numpy((rng.standard_normal((1, 2 * k)) * 3).astype(np.float32))
    act = _C.Tensor.empty((1, k), "float32")
    _lib.check(lib.gq_swiglu(ctx, gu.storage.handle, 1, k, act.storage.handle))
    want = w.linear(act, None, _lib.KERNEL_IMMA).numpy()
    assert np.abs(w.linear_swiglu(gu).numpy() - want).max() <= 2e-6 * np.abs(want).max()  # hardware exp2 and reciprocal in the prologue


def test_fused_linears_refuse_row_lengths_that_are_not_multiples_of_four():
    _C, _lib, lib, ctx = _env()
    w = _C.Int8Weight.quantize(_C.Tensor.from_numpy(np.ones((3, 6), dtype=np.float32)))
    x = _C.Tensor.from_numpy(np.ones((1, 6), dtype=np.float32))
    with pytest.raises(RuntimeError, match="multiple of 4"):
        w.linear_norm(x, None, x, 1e-6)


@pytest.mark.parametrize("dim,heads,kv_heads,max_len,length", [(64, 14, 2, 1024, 1023), (64, 14, 2, 1024, 0), (64, 14, 2, 1024, 1024),
                                                               (32, 4, 2, 48, 20), (128, 8, 4, 300, 37), (64, 4, 1, 2500, 1700)])
def test_rope_attention_in_one_launch_equals_the_two_operators(dim, heads, kv_heads, max_len, length):
    """gq_attn_decode_rope == gq_rope_kv_append then gq_attn_decode: same output, same cache afterwards."""
    _C, _lib, lib, ctx = _env()
    rng = np.random.default_rng(dim + length + heads)
    k = rng.standard_normal(kv_heads * max_len * dim).astype(np.float32)
    v = rng.standard_normal(kv_heads * max_len * dim).astype(np.float32)
    qkv = rng.standard_normal((heads + 2 * kv_heads) * dim).astype(np.float32)
    ang = rng.uniform(0, 6.28, (max_len, dim)).astype(np.float32)
    cos, sin = _C.Tensor.from_numpy(np.cos(ang)), _C.Tensor.from_numpy(np.sin(ang))
    lens = _C.Tensor.from_numpy(np.array([length, 7], dtype=np.int32))
    nbytes = ctypes.c_uint64()
    _lib.check(lib.gq_attn_scratch_bytes(ctx, heads, dim, max_len, ctypes.byref(nbytes)))
    scratch = _C.Tensor.from_numpy(np.zeros(nbytes.value // 4, dtype=np.float32))
    tq = _C.Tensor.from_numpy(qkv)
    k1, v1, k2, v2 = (_C.Tensor.from_numpy(a) for a in (k, v, k, v))
    q = _C.Tensor.empty((heads * dim,), "float32")
    want, got = _C.Tensor.empty((heads, dim), "float32"), _C.Tensor.empty((heads, dim), "float32")
    _lib.check(lib.gq_rope_kv_append(ctx, tq.storage.handle, cos.storage.handle, sin.storage.handle, lens.storage.handle, 0, 2, heads, kv_heads,
                                     dim, max_len, q.storage.handle, k1.storage.handle, 0, v1.storage.handle, 0))
    _lib.check(lib.gq_attn_decode(ctx, q.storage.handle, k1.storage.handle, 0, v1.storage.handle, 0, lens.storage.handle, 0, 2, heads,
                                  kv_heads, dim, max_len, dim ** -0.5, scratch.storage.handle, want.storage.handle))
    _lib.check(lib.gq_attn_decode_rope(ctx, tq.storage.handle, cos.storage.handle, sin.storage.handle, k2.storage.handle, 0, v2.storage.handle,
                                       0, lens.storage.handle, 0, 2, heads, kv_heads, dim, max_len, dim ** -0.5, scratch.storage.handle,
                                       got.storage.handle))
    np.testing.assert_array_equal(k2.numpy(), k1.numpy())
    np.testing.assert_array_equal(v2.numpy(), v1.numpy())
    if length < max_len:
        assert not np.array_equal(k1.numpy(), k)  # something was appended
    np.testing.assert_array_equal(got.numpy(), want.numpy())
