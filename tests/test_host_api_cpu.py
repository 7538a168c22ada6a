"""Host-side logic that needs no device: configs and their refusals, the int4
host packer, the safetensors reader's widening, graphed's signature keys."""
import json
import struct

import numpy as np
import pytest

import oracle
from grilly2_b200.infer import quantization as Q
from grilly2_b200.infer import safetensors as S


def test_config_refusals_match_the_reference():
    """tests/python/test_quantization.py:142-153, :236-239."""
    assert Q.Int8WeightOnlyConfig().granularity == Q.PerRow()
    with pytest.raises(AssertionError, match="group_size"):
        Q.Int8WeightOnlyConfig(group_size=32)
    with pytest.raises(ValueError, match="version 1"):
        Q.Int8WeightOnlyConfig(version=1)
    with pytest.raises(NotImplementedError, match="granularity"):
        Q.Int8WeightOnlyConfig(granularity=Q.PerRow(dim=0))
    with pytest.raises(ValueError, match="multiple of 32"):
        Q.Int4WeightOnlyConfig(group_size=30)
    with pytest.raises(ValueError, match="version 1"):
        Q.Int4WeightOnlyConfig(version=1)
    with pytest.raises(TypeError, match="from_hp"):
        Q.Int8Tensor(None)

    class Empty:
        def named_modules(self):
            return iter(())

    with pytest.raises(NotImplementedError, match="quantize_ with"):
        Q.quantize_(Empty(), object())
    with pytest.raises(NotImplementedError, match="device 'cuda'"):
        Q.quantize_(Empty(), Q.Int8WeightOnlyConfig(), device="cuda")
    Q.quantize_(Empty(), Q.Int8WeightOnlyConfig(), device="cpu")  # the alias is accepted


def test_from_parts_packer_equals_the_oracle_packer():
    rng = np.random.default_rng(0)
    for n, k in [(3, 32), (2, 130), (4, 896)]:
        levels = rng.integers(0, 16, (n, k)).astype(np.uint8)
        words = -(-k // 32) * 4
        padded = np.zeros((n, words * 8), dtype=np.uint32)
        padded[:, :k] = levels
        shifts = (4 * np.arange(8, dtype=np.uint32))[None, None, :]
        packed = np.bitwise_or.reduce(padded.reshape(n, words, 8) << shifts, axis=2).astype(np.uint32)
        np.testing.assert_array_equal(packed, oracle.pack_levels_q4(levels))


def write_safetensors(path, tensors):
    header, blobs, off = {}, [], 0
    for name, (dtype, arr) in tensors.items():
        raw = arr.tobytes()
        header[name] = {"dtype": dtype, "shape": list(arr.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    h = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + b"".join(blobs))


def test_widening_is_exact_for_every_16_bit_pattern():
    """All 65,536 bf16 and f16 patterns widen bit for bit
    (crates/grilly-infer/tests/safetensors.rs; docs/inference.md:69-78)."""
    import torch
    pats = np.arange(65536, dtype=np.uint16)
    got = S._widen(pats.view(np.uint8), "BF16", (65536,))
    want = torch.from_numpy(pats.view(np.int16)).view(torch.bfloat16).float().numpy()
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))
    got = S._widen(pats.view(np.uint8), "F16", (65536,))
    want = torch.from_numpy(pats.view(np.int16)).view(torch.float16).float().numpy()
    finite = ~np.isnan(want)  # NaN payloads differ only in the quiet bit between converters
    np.testing.assert_array_equal(got.view(np.uint32)[finite], want.view(np.uint32)[finite])
    assert np.isnan(got[~finite]).all()


def test_reader_orders_and_bounds(tmp_path):
    p = tmp_path / "a.safetensors"
    write_safetensors(p, {"b": ("F32", np.arange(6, dtype=np.float32).reshape(2, 3)),
                          "a": ("I64", np.arange(4, dtype=np.int64))})
    with S.safe_open(p) as f:
        assert f.keys() == ["a", "b"] and f.offset_keys() == ["b", "a"]
        assert f.get_slice_shape("b") == (2, 3)
    bad = tmp_path / "bad.safetensors"
    bad.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(RuntimeError, match="exceeds the file"):
        S.safe_open(bad)


def test_graphed_signatures():
    from grilly2_b200 import _graph
    assert _graph._signature((1, "a", None)) != _graph._signature((2, "a", None))
    assert _graph._signature([1]) != _graph._signature((1,))
