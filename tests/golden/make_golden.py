"""Generates tests/golden/*.npz. Run in the build container, where the
reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/reference

What it pins, and with what:

* int4_rtn.npz — the reference's OWN code: python/grilly/infer/gptq.py's
  ``rtn_quantize`` (numpy only, loaded by file path) run on the weight list of
  crates/grilly-infer/tests/quant4.rs:89-96, drawn with that test's seeded
  xorshift generator, plus a normal(0, 0.02) weight of the benchmark's kind.
* int8_formula.npz / int4_formula.npz — the torch formulas the reference's
  tests use as their oracle (tests/python/test_quantization.py:38-43 and
  :172-190), evaluated by torch here, on the shape list and edge cases of
  crates/grilly-infer/tests/quant.rs:62-83 (an all-zero row; a row whose
  extremes land on +-127.5 and a tie at 0.5), with the inputs drawn by that
  test's own seeded xorshift generator and seeds (quant.rs:27-37, seed
  n * 1000 + k, range [-3, 3]): the vectors the reference's test holds. The
  reference's host `reference()` (quant.rs:40-53), restated in numpy float32,
  is evaluated beside the torch formula and must agree bit for bit.

The arrays are stored with their inputs, so the tests need neither the
reference nor torch.
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import xorshift_data  # noqa: E402  (the seeded generator only)


def load_gptq(reference_root):
    path = os.path.join(reference_root, "python", "grilly", "infer", "gptq.py")
    spec = importlib.util.spec_from_file_location("ref_gptq", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def int8_formula(w):
    w = torch.from_numpy(w)
    amax = torch.maximum(-torch.clamp(w.amin(dim=1), max=0), torch.clamp(w.amax(dim=1), min=0))
    scale = torch.clamp(amax / 127.5, min=torch.finfo(torch.float32).eps)
    q = torch.clamp(torch.round(w * (1.0 / scale[:, None])), -128, 127).to(torch.int8)
    deq = q.float() * scale[:, None]
    return q.numpy(), scale.numpy(), deq.numpy()


def int4_formula(w, group):
    w = torch.from_numpy(w)
    rows, k = w.shape
    groups = (k + group - 1) // group
    padded = torch.nn.functional.pad(w, (0, groups * group - k), value=float("nan"))
    blocks = padded.reshape(rows, groups, group)
    lo = blocks.nan_to_num(float("inf")).amin(dim=2)
    hi = blocks.nan_to_num(float("-inf")).amax(dim=2)
    scale = torch.clamp((hi - lo) / 15.0, min=torch.finfo(torch.float32).eps)
    zero = lo + 8.0 * scale
    levels = torch.clamp(torch.round((blocks - lo[..., None]) / scale[..., None]), 0, 15)
    return levels.reshape(rows, -1)[:, :k].to(torch.uint8).numpy(), scale.numpy(), zero.numpy()


def int8_host_reference(w):
    """The reference's own host check, crates/grilly-infer/tests/quant.rs:40-53 (`reference`), statement for statement in
    numpy float32: amax by fold of |v|, scale = max(amax / 127.5, eps), inv = 1 / scale, q = clamp(round_ties_even(v * inv))."""
    f32 = np.float32
    amax = np.abs(w).max(axis=1).astype(f32)
    scale = np.maximum(amax / f32(127.5), np.finfo(f32).eps).astype(f32)
    inv = (f32(1.0) / scale).astype(f32)
    q = np.clip(np.rint((w * inv[:, None]).astype(f32)), -128.0, 127.0).astype(np.int8)
    return q, scale


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/the/reference/checkout")
    ref = sys.argv[1]
    gptq = load_gptq(ref)

    out = {}
    cases = [(1, 32, 32), (3, 128, 128), (5, 130, 128), (2, 256, 64), (7, 896, 128), (4, 4864, 128)]
    for i, (n, k, group) in enumerate(cases):
        w = xorshift_data(n * k, n + k + group, -1.5, 1.0, int4_form=True).reshape(n, k)
        levels, scales, zeros = gptq.rtn_quantize(w, group)
        out.update({f"w{i}": w, f"group{i}": np.int64(group), f"levels{i}": levels, f"scale{i}": scales,
                    f"zero{i}": zeros})
    i = len(cases)
    w = (np.random.default_rng(1).standard_normal((16, 4096)) * 0.02).astype(np.float32)
    levels, scales, zeros = gptq.rtn_quantize(w, 128)
    out.update({f"w{i}": w, f"group{i}": np.int64(128), f"levels{i}": levels, f"scale{i}": scales, f"zero{i}": zeros})
    out["count"] = np.int64(i + 1)
    np.savez_compressed(os.path.join(HERE, "int4_rtn.npz"), **out)

    out = {}
    shapes = [(1, 1), (3, 5), (5, 17), (4, 16), (7, 33), (64, 896), (9, 4864)]
    for i, (n, k) in enumerate(shapes):
        w = xorshift_data(n * k, n * 1000 + k, -3.0, 3.0).reshape(n, k)
        w[0] = 0.0
        if n > 2:
            w[2, 0] = 2.55
            if k > 1:
                w[2, 1] = -2.55
            if k > 2:
                w[2, 2] = 0.01
        q, scale, deq = int8_formula(w)
        q_host, scale_host = int8_host_reference(w)  # two independent statements of the reference's check must agree
        assert np.array_equal(q, q_host) and np.array_equal(scale.view(np.uint32), scale_host.view(np.uint32)), (n, k)
        out.update({f"w{i}": w, f"q{i}": q, f"scale{i}": scale, f"deq{i}": deq})
    out["count"] = np.int64(len(shapes))
    np.savez_compressed(os.path.join(HERE, "int8_formula.npz"), **out)

    out = {}
    rng = np.random.default_rng(3)
    j = 0
    for group in (32, 64, 128):
        for rows, k in [(4, 128), (3, 896), (2, 4864), (5, 130)]:
            w = rng.standard_normal((rows, k)).astype(np.float32)
            levels, scale, zero = int4_formula(w, group)
            out.update({f"w{j}": w, f"group{j}": np.int64(group), f"levels{j}": levels, f"scale{j}": scale,
                        f"zero{j}": zero})
            j += 1
    out["count"] = np.int64(j)
    np.savez_compressed(os.path.join(HERE, "int4_formula.npz"), **out)
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))


if __name__ == "__main__":
    main()
