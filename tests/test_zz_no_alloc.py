"""gq_attn_decode_static — decode attention whose scratch is a fixed array in the library's device memory —
against gq_attn_decode on the same inputs, through the C ABI. Collected last; passes alone or after the rest."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _case(seed, heads, kv_heads, dim, max_len, length):
    from grilly2_b200 import _C
    rng = np.random.default_rng(seed)
    k = rng.standard_normal(kv_heads * max_len * dim).astype(np.float32)
    v = rng.standard_normal(kv_heads * max_len * dim).astype(np.float32)
    q = rng.standard_normal((heads, dim)).astype(np.float32)
    lens = np.array([length, 3], dtype=np.int32)
    return tuple(_C.Tensor.from_numpy(a) for a in (q, k, v, lens))


def test_static_scratch_attention_equals_the_buffer_one_twice_in_a_row():
    from grilly2_b200 import _C, _lib
    lib, ctx = _lib.load(), _C.context()
    heads, kv_heads, dim, max_len = 14, 2, 64, 1024
    nbytes = ctypes.c_uint64()
    _lib.check(lib.gq_attn_scratch_bytes(ctx, heads, dim, max_len, ctypes.byref(nbytes)))
    scratch = _C.Tensor.from_numpy(np.zeros(nbytes.value // 4, dtype=np.float32))
    import torch
    torch.cuda.mem_get_info()  # torch's own context exists from here on, so it cannot show up as a difference below
    # one warm call first: the very first launch of a kernel makes the driver load its code, which is set-up, not the call's doing
    q, k, v, lens = _case(39, heads, kv_heads, dim, max_len, 100)
    warm = _C.Tensor.empty((heads, dim), "float32")
    _lib.check(lib.gq_attn_decode_static(ctx, q.storage.handle, k.storage.handle, 0, v.storage.handle, 0, lens.storage.handle, 0, 2,
                                         heads, kv_heads, dim, max_len, dim ** -0.5, warm.storage.handle))
    before = _C.submit_stats()
    for call, length in enumerate((1023, 517)):  # two calls in a row: the shared array must be reusable as it is left
        q, k, v, lens = _case(40 + call, heads, kv_heads, dim, max_len, length)
        want, got = _C.Tensor.empty((heads, dim), "float32"), _C.Tensor.empty((heads, dim), "float32")
        allocs = _C.submit_stats()["buffer_allocations"]
        _C.synchronize()
        free_before = torch.cuda.mem_get_info()[0]  # the driver's own count of free device memory: an observation, not a self-report
        _lib.check(lib.gq_attn_decode_static(ctx, q.storage.handle, k.storage.handle, 0, v.storage.handle, 0, lens.storage.handle, 0, 2,
                                             heads, kv_heads, dim, max_len, dim ** -0.5, got.storage.handle))
        _C.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, "device memory was allocated during the call"
        assert _C.submit_stats()["buffer_allocations"] == allocs
        _lib.check(lib.gq_attn_decode(ctx, q.storage.handle, k.storage.handle, 0, v.storage.handle, 0, lens.storage.handle, 0, 2,
                                      heads, kv_heads, dim, max_len, dim ** -0.5, scratch.storage.handle, want.storage.handle))
        w = want.numpy()
        assert np.isfinite(w).all() and np.abs(w).max() > 0
        np.testing.assert_array_equal(got.numpy(), w)
    assert _C.submit_stats()["launches"] == before["launches"] + 4


def test_static_scratch_attention_replays_inside_a_graph():
    """Captured after one eager call (the first call on a device looks the array up): every replay equals the buffer form."""
    from grilly2_b200 import _C, _lib
    lib, ctx = _lib.load(), _C.context()
    heads, kv_heads, dim, max_len = 14, 2, 64, 256
    nbytes = ctypes.c_uint64()
    _lib.check(lib.gq_attn_scratch_bytes(ctx, heads, dim, max_len, ctypes.byref(nbytes)))
    scratch = _C.Tensor.from_numpy(np.zeros(nbytes.value // 4, dtype=np.float32))
    q, k, v, lens = _case(77, heads, kv_heads, dim, max_len, 200)
    got, want = _C.Tensor.empty((heads, dim), "float32"), _C.Tensor.empty((heads, dim), "float32")

    def static_call():
        _lib.check(lib.gq_attn_decode_static(ctx, q.storage.handle, k.storage.handle, 0, v.storage.handle, 0, lens.storage.handle, 0, 2,
                                             heads, kv_heads, dim, max_len, dim ** -0.5, got.storage.handle))

    static_call()
    _C.begin_capture()
    static_call()
    graph = _C.end_capture()
    for length in (200, 31, 256):
        lens.copy_(_C.Tensor.from_numpy(np.array([length, 3], dtype=np.int32)))
        q.copy_(_C.Tensor.from_numpy(np.random.default_rng(length).standard_normal((heads, dim)).astype(np.float32)))
        graph.replay()
        _lib.check(lib.gq_attn_decode(ctx, q.storage.handle, k.storage.handle, 0, v.storage.handle, 0, lens.storage.handle, 0, 2,
                                      heads, kv_heads, dim, max_len, dim ** -0.5, scratch.storage.handle, want.storage.handle))
        np.testing.assert_array_equal(got.numpy(), want.numpy())


def test_static_scratch_attention_refuses_what_does_not_fit():
    from grilly2_b200 import _C, _lib
    lib, ctx = _lib.load(), _C.context()
    t = _C.Tensor.from_numpy(np.zeros(16, dtype=np.float32))
    ti = _C.Tensor.from_numpy(np.zeros(1, dtype=np.int32))
    # 64 heads x 79 splits x 130 floats = 2.6 MB of partial results: beyond the fixed 2 MiB
    rc = lib.gq_attn_decode_static(ctx, t.storage.handle, t.storage.handle, 0, t.storage.handle, 0, ti.storage.handle, 0, 1, 64, 8, 128,
                                   40000, 1.0, t.storage.handle)
    assert rc != 0
    assert "beyond the fixed" in _lib.last_error()
