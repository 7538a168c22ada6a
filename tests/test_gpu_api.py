"""The Python surface on a GPU: quantize_ / load_quantized_ / persistent-memory
accounting / graphed, mirroring the reference's Python tests
(tests/python/test_quantization.py, test_load_quantized.py, test_graph.py)."""
import gc

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def g():
    import grilly2_b200 as g
    return g


def test_quantize_api_as_torchaos(g):
    import grilly2_b200.nn as gnn
    from grilly2_b200.infer.quantization import Int4Tensor, Int4WeightOnlyConfig, Int8Tensor, Int8WeightOnlyConfig, quantize_
    model = gnn.Sequential(gnn.Linear(8, 8), gnn.Linear(8, 4))
    quantize_(model, Int8WeightOnlyConfig(), filter_fn=lambda m, name: name == "1")
    assert not isinstance(model[0].weight, Int8Tensor) and isinstance(model[1].weight, Int8Tensor)
    first = model[1].weight
    quantize_(model, Int8WeightOnlyConfig())  # the default filter skips weights already quantized
    assert model[1].weight is first and isinstance(model[0].weight, Int8Tensor)
    assert tuple(first.shape) == (4, 8) and first.dtype is g.float32 and first.numel() == 32
    assert "Int8Tensor(shape=(4, 8)" in repr(first)
    assert sum(p.numel() for p in model.parameters()) == 8 * 8 + 8 + 4 * 8 + 4
    assert first.requires_grad is False and first.grad is None
    with pytest.raises(RuntimeError, match="frozen"):
        first.requires_grad_(True)
    with pytest.raises(NotImplementedError, match="device 'cuda'"):
        quantize_(model, Int8WeightOnlyConfig(), device="cuda")

    m4 = gnn.Sequential(gnn.Linear(64, 32))
    quantize_(m4, Int4WeightOnlyConfig(group_size=32))
    assert isinstance(m4[0].weight, Int4Tensor) and not isinstance(m4[0].weight, Int8Tensor)
    assert m4[0].weight.group_size == 32 and "group_size=32" in repr(m4[0].weight)
    quantize_(m4, Int8WeightOnlyConfig())
    assert isinstance(m4[0].weight, Int4Tensor)
    # the quantized nn.Linear forward is the oracle's linear of the same weight
    x = np.random.default_rng(0).standard_normal((3, 64)).astype(np.float32)
    w = m4[0].weight.dequantize().numpy()
    y = m4(g.from_numpy(x)).numpy()
    assert np.abs(y - (x @ w.T + m4[0].bias.numpy())).max() < 1e-4


def test_quantized_weights_are_counted_in_persistent_memory(g):
    """tests/python/test_quantization.py:156-166: Linear(900, 70) pads rows to
    912 bytes; the float weight is freed when it is replaced."""
    import grilly2_b200.nn as gnn
    from grilly2_b200 import _C
    from grilly2_b200.infer.quantization import Int8WeightOnlyConfig, quantize_

    def persistent():
        gc.collect()
        return _C.submit_stats()["persistent_bytes"]

    before = persistent()
    lin = gnn.Linear(900, 70)
    assert persistent() - before == 4 * (900 * 70 + 70)
    quantize_(lin, Int8WeightOnlyConfig())
    assert lin.weight.nbytes == 70 * 912 + 70 * 4
    assert persistent() - before == lin.weight.nbytes + 4 * 70  # the float weight is freed; the bias stays


def test_streamed_load_equals_load_then_quantize(g, tmp_path):
    """tests/python/test_load_quantized.py:58-119."""
    import torch
    from safetensors.torch import save_file
    import grilly2_b200.nn as gnn
    from grilly2_b200.infer.quantization import (Int4WeightOnlyConfig, Int8Tensor, Int8WeightOnlyConfig,
                                                 load_quantized_, quantize_)
    torch.manual_seed(0)
    sd = {"0.weight": torch.randn(48, 64), "0.bias": torch.randn(48), "1.weight": torch.randn(16, 48).bfloat16(),
          "1.bias": torch.randn(16)}
    path = str(tmp_path / "m.safetensors")
    save_file(sd, path)

    def make():
        return gnn.Sequential(gnn.Linear(64, 48), gnn.Linear(48, 16))

    for config in (Int8WeightOnlyConfig(), Int4WeightOnlyConfig(group_size=32)):
        streamed = make()
        names = load_quantized_(streamed, path, config)
        assert names == set(sd)
        two_step = make()
        two_step.load_state_dict({k: g.from_numpy(v.float().numpy()) for k, v in sd.items()})
        quantize_(two_step, config)
        for a, b in zip(streamed.parameters(), two_step.parameters()):
            assert type(a) is type(b)
            if hasattr(a, "_q"):
                np.testing.assert_array_equal(a._q.packed().numpy(), b._q.packed().numpy())
                np.testing.assert_array_equal(a.scale.numpy().view(np.uint32), b.scale.numpy().view(np.uint32))
            else:
                np.testing.assert_array_equal(a.numpy(), b.numpy())
    assert isinstance(streamed[0].weight, Int8Tensor) is False
    # keep_vars=True does not dequantize (test_load_quantized.py:145-160)
    kept = streamed.state_dict(keep_vars=True)
    assert hasattr(kept["0.weight"], "_q") and not hasattr(streamed.state_dict()["0.weight"], "_q")

    wrong = gnn.Sequential(gnn.Linear(64, 48), gnn.Linear(48, 16), gnn.Linear(16, 4))
    with pytest.raises(RuntimeError, match='Missing key.*"2.weight"'):
        load_quantized_(wrong, path, Int8WeightOnlyConfig())
    small = gnn.Sequential(gnn.Linear(64, 48))
    with pytest.raises(RuntimeError, match='Unexpected key.*"1.weight"'):
        load_quantized_(small, path, Int8WeightOnlyConfig())
    load_quantized_(small, path, Int8WeightOnlyConfig(), strict=False)
    misfit = gnn.Sequential(gnn.Linear(64, 48), gnn.Linear(48, 8))
    with pytest.raises(RuntimeError, match="size mismatch for 1.weight"):
        load_quantized_(misfit, path, Int8WeightOnlyConfig())


def test_streaming_peak_is_one_float_tensor(g, tmp_path):
    """tests/python/test_load_quantized.py:90-96: the persistent peak while
    streaming stays below twice the largest tensor plus what ends up resident."""
    import torch
    from safetensors.torch import save_file
    import grilly2_b200.nn as gnn
    from grilly2_b200 import _C
    from grilly2_b200.infer.quantization import Int8WeightOnlyConfig, load_quantized_
    sd = {f"{i}.weight": torch.randn(256, 256) for i in range(6)}
    path = str(tmp_path / "big.safetensors")
    save_file(sd, path)
    gc.collect()
    empty = _C.submit_stats()["persistent_bytes"]
    model = gnn.Sequential(*[gnn.Linear(256, 256, bias=False) for _ in range(6)])
    gc.collect()
    _C.reset_persistent_peak()
    base = _C.submit_stats()["persistent_bytes"]
    assert base - empty == 6 * 256 * 256 * 4
    load_quantized_(model, path, Int8WeightOnlyConfig())
    gc.collect()
    stats = _C.submit_stats()
    resident = sum(p.nbytes for p in model.parameters())
    assert stats["persistent_bytes"] - empty == resident  # every float weight is gone
    # at most one float tensor from the file (plus its quantized copy) is alive beside the model
    assert stats["persistent_peak"] - base <= 2 * 256 * 256 * 4


def test_graphed_replays_bit_exactly(g):
    """tests/python/test_graph.py: first sighting eager, second captured, then
    replays; replay == eager; the same output objects come back; a host read
    inside a capture is refused."""
    import grilly2_b200.nn.functional as F
    from grilly2_b200 import _C
    from grilly2_b200.infer.quantization import Int4Tensor, Int8Tensor
    rng = np.random.default_rng(2)
    w1 = Int8Tensor.from_hp(g.from_numpy(rng.standard_normal((256, 128)).astype(np.float32)))
    w2 = Int4Tensor.from_hp(g.from_numpy(rng.standard_normal((64, 256)).astype(np.float32)), 64)

    def step(x):
        return F.linear(F.linear(x, w1), w2)

    fast = g.graphed(step)
    xs = [rng.standard_normal((1, 128)).astype(np.float32) for _ in range(5)]
    eager = [step(g.from_numpy(x)).numpy() for x in xs]
    before = _C.submit_stats()
    outs = []
    for x in xs:
        outs.append(fast(g.from_numpy(x)))
        np.testing.assert_array_equal(outs[-1].numpy(), eager[len(outs) - 1])
    after = _C.submit_stats()
    assert (fast.misses, fast.captures, fast.replays, fast.graphs) == (1, 1, 3, 1)
    assert outs[2] is outs[3] is outs[4]
    assert after["graph_launches"] - before["graph_launches"] == 3
    assert "CommandGraph(commands=" in repr(next(iter(fast.captured.values())).graph)

    def reads_back(x):
        y = F.linear(x, w1)
        y.numpy()
        return y

    bad = g.graphed(reads_back)
    bad(g.from_numpy(xs[0]))
    with pytest.raises(RuntimeError, match="read data back"):
        bad(g.from_numpy(xs[0]))
    assert not _C.capturing()
    step(g.from_numpy(xs[0])).numpy()  # the context still works

    def nothing(x):
        return x

    empty = g.graphed(nothing)
    empty(g.from_numpy(xs[0]))
    with pytest.raises(RuntimeError, match="nothing was captured"):
        empty(g.from_numpy(xs[0]))


def test_misuse_is_reported_not_thrown(g):
    """crates/grilly-sys/tests/gpu.rs:272-329: every misuse is GQ_ERR + message."""
    import ctypes
    from grilly2_b200 import _C, _lib
    lib, ctx = _lib.load(), _C.context()
    assert lib.gq_buffer_release(ctx, 0) == _lib.GQ_ERR and "invalid buffer handle" in _lib.last_error()
    assert lib.gq_buffer_release(ctx, 1 << 60) == _lib.GQ_ERR
    h = ctypes.c_uint64()
    assert lib.gq_buffer_create(ctx, 64, 7, ctypes.byref(h)) == _lib.GQ_ERR and "memory class" in _lib.last_error()
    assert lib.gq_buffer_create(ctx, 64, 0, ctypes.byref(h)) == _lib.GQ_OK
    small = h.value
    # a weight of 4 x 16 floats does not fit 64 bytes
    assert lib.gq_int8_quantize(ctx, small, 0, 4, 16, small, small) == _lib.GQ_ERR
    assert "buffer holds 64 bytes" in _lib.last_error()
    assert lib.gq_int4_quantize(ctx, small, 0, 1, 16, 48, small, small, small) == _lib.GQ_ERR
    assert "multiple of 32" in _lib.last_error()
    assert lib.gq_int8_linear(ctx, small, 0, 1, 16, small, small, 0, 0, 1, small, 9) == _lib.GQ_ERR
    assert lib.gq_download(ctx, small, 60, None, 8) == _lib.GQ_ERR
    assert lib.gq_end_capture(ctx, None) == _lib.GQ_ERR and "no capture is running" in _lib.last_error()
    assert lib.gq_buffer_release(ctx, small) == _lib.GQ_OK
    assert lib.gq_buffer_release(ctx, small) == _lib.GQ_ERR  # released twice
    assert lib.gq_synchronize(ctx) == _lib.GQ_OK  # and the context is still usable
