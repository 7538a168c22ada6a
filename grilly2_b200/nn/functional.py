"""``F.linear`` with the hook quantized weights use
(python/grilly/nn/functional.py:21-29)."""
from __future__ import annotations


def linear(input, weight, bias=None):
    """``input @ weight.T + bias`` over the last dimension of ``input``.

    A weight whose type defines ``_grilly_linear`` brings its own kernel — the
    quantized ones do. The float32 matmul is outside this backend: it is the
    reference's float path, not the quantized one this library replaces."""
    own = getattr(type(weight), "_grilly_linear", None)
    if own is not None:
        return own(weight, input, bias)
    raise NotImplementedError(
        "grilly: F.linear with a float32 weight is not implemented yet (this backend runs the weight-only "
        "quantized linears; call quantize_(model, Int8WeightOnlyConfig()) or load_quantized_ first)")
