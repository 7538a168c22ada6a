"""Inference-side API of the quantized path: ``quantization`` and the
streaming ``safetensors`` loader."""
from . import quantization, safetensors  # noqa: F401
