"""Quantizing the parts of a fused projection straight into the fused weight, and the pre-packed checkpoint: what the
reference names as its next step (docs/inference.md:900-904). Bit-exact throughout."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_fused_quantization_equals_cat_bit_for_bit_and_never_holds_the_parts_twice():
    from grilly2_b200 import _C
    rng = np.random.default_rng(3)
    parts = [(rng.standard_normal((n, 896)) * 0.02).astype(np.float32) for n in (896, 128, 128)]
    x = _C.Tensor.from_numpy(rng.standard_normal((1, 896)).astype(np.float32))
    for bits in (8, 4):
        ts = [_C.Tensor.from_numpy(p) for p in parts]
        _C.synchronize()
        base = _C.submit_stats()["persistent_bytes"]
        _C.reset_persistent_peak()
        fused = _C.Int8Weight.quantize_fused(ts) if bits == 8 else _C.Int4Weight.quantize_fused(ts, 128)
        peak_direct = _C.submit_stats()["persistent_peak"] - base
        assert peak_direct == fused.nbytes  # exactly one copy of the quantized data ever existed
        _C.reset_persistent_peak()
        base = _C.submit_stats()["persistent_bytes"]
        apart = [_C.Int8Weight.quantize(t) if bits == 8 else _C.Int4Weight.quantize(t, 128) for t in ts]
        catted = (_C.Int8Weight if bits == 8 else _C.Int4Weight).cat(apart)
        assert _C.submit_stats()["persistent_peak"] - base == 2 * fused.nbytes  # the route it replaces holds them twice
        np.testing.assert_array_equal(fused.packed().numpy(), catted.packed().numpy())
        np.testing.assert_array_equal(fused.scale().numpy().view(np.uint32), catted.scale().numpy().view(np.uint32))
        if bits == 4:
            np.testing.assert_array_equal(fused.zero().numpy().view(np.uint32), catted.zero().numpy().view(np.uint32))
        np.testing.assert_array_equal(fused.linear(x).numpy(), catted.linear(x).numpy())
        assert fused.shape == (1152, 896)
        del fused, apart, catted, ts  # the next round's byte counts start from a clean slate


def test_quantize_rows_refuses_what_does_not_fit():
    import ctypes
    from grilly2_b200 import _C, _lib
    lib, ctx = _lib.load(), _C.context()
    w = _C.Tensor.from_numpy(np.ones((4, 32), np.float32))
    q = _C.Tensor.empty((6, 8), "int32", persistent=True)
    s = _C.Tensor.empty((6,), "float32", persistent=True)
    assert lib.gq_int8_quantize_rows(ctx, w.storage.handle, 0, 4, 32, q.storage.handle, s.storage.handle, 3, 6) == _lib.GQ_ERR
    assert "do not fit" in _lib.last_error()
    assert lib.gq_int8_quantize_rows(ctx, w.storage.handle, 0, 4, 32, q.storage.handle, s.storage.handle, 2, 6) == _lib.GQ_OK


@pytest.mark.parametrize("bits", [8, 4])
def test_a_prepacked_checkpoint_round_trips_without_a_float_copy(tmp_path, bits):
    import grilly2_b200 as g
    import grilly2_b200.nn as nn
    from grilly2_b200 import _C
    from grilly2_b200.infer.quantization import (Int4Tensor, Int4WeightOnlyConfig, Int8Tensor, Int8WeightOnlyConfig, load_packed_,
                                                 quantize_, save_packed)
    rng = np.random.default_rng(bits)

    def make():
        m = nn.Sequential(nn.Linear(256, 96, bias=True), nn.Linear(96, 40, bias=False))
        return m

    src = make()
    for p in src.parameters():
        p.copy_(g.from_numpy((rng.standard_normal(tuple(p.shape)) * 0.05).astype(np.float32)))
    quantize_(src, Int8WeightOnlyConfig() if bits == 8 else Int4WeightOnlyConfig(group_size=32))
    path = tmp_path / "packed.safetensors"
    names = save_packed(src, path)
    assert "0.weight.__q" in names and "0.bias" in names and ("0.weight.__zero" in names) == (bits == 4)

    dst = make()
    _C.synchronize()
    base = _C.submit_stats()["persistent_bytes"]
    _C.reset_persistent_peak()
    got = load_packed_(dst, path)
    assert got == {"0.weight", "0.bias", "1.weight"}
    kind = Int8Tensor if bits == 8 else Int4Tensor
    assert isinstance(dst[0].weight, kind) and isinstance(dst[1].weight, kind)
    for a, b in ((src[0], dst[0]), (src[1], dst[1])):
        np.testing.assert_array_equal(a.weight._q.packed().numpy(), b.weight._q.packed().numpy())
        np.testing.assert_array_equal(a.weight._q.scale().numpy().view(np.uint32), b.weight._q.scale().numpy().view(np.uint32))
        if bits == 4:
            np.testing.assert_array_equal(a.weight._q.zero().numpy().view(np.uint32), b.weight._q.zero().numpy().view(np.uint32))
            assert b.weight.group_size == 32
    np.testing.assert_array_equal(src[0].bias.numpy(), dst[0].bias.numpy())
    x = g.from_numpy(rng.standard_normal((3, 256)).astype(np.float32))
    np.testing.assert_array_equal(dst(x).numpy(), src(x).numpy())
    # what stayed on the device after the load is the packed data and the bias: no float32 weight was ever uploaded
    held = sum(m.weight.nbytes for m in (dst[0], dst[1])) + 96 * 4
    float_weights = (256 * 96 + 96 * 40) * 4
    assert _C.submit_stats()["persistent_peak"] - base < held + float_weights // 4

    with pytest.raises(RuntimeError, match="not a pre-packed checkpoint"):
        from safetensors.numpy import save_file
        plain = tmp_path / "plain.safetensors"
        save_file({"0.weight": np.zeros((96, 256), np.float32)}, str(plain))
        load_packed_(make(), plain)
