"""CPU-side checks of the boundary: libgq.so builds, loads and exports every
symbol include/gq.h declares; the ctypes prototypes cover the header; and
without a GPU the library reports an error instead of falling back."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "gq.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gq_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = declared_functions()
    for must in ["gq_create", "gq_destroy", "gq_last_error", "gq_int8_quantize", "gq_int8_linear", "gq_int8_dequantize",
                 "gq_int4_quantize", "gq_int4_linear", "gq_int4_dequantize", "gq_begin_capture", "gq_end_capture",
                 "gq_graph_replay", "gq_buffer_create", "gq_upload", "gq_download", "gq_stats_get"]:
        assert must in names


def test_library_exports_every_declared_symbol():
    from grilly2_b200 import _lib
    lib = _lib.load()
    for name in declared_functions():
        assert getattr(lib, name) is not None, name


def test_ctypes_prototypes_cover_the_header():
    from grilly2_b200 import _lib
    bound = set(_lib.PROTOTYPES) | set(_lib.VOID_FUNCTIONS) | {"gq_last_error"}
    assert set(declared_functions()) == bound


def test_kernel_selectors_match_the_header():
    """The host mirror's KERNEL_* constants are the header's GQ_KERNEL_* macros, every one of them."""
    from grilly2_b200 import _lib
    text = open(os.path.join(ROOT, "include", "gq.h")).read()
    macros = {name: int(value) for name, value in re.findall(r"#define\s+GQ_(KERNEL_[A-Z0-9_]+)\s+(\d+)", text)}
    assert len(macros) >= 9 and len(set(macros.values())) == len(macros)
    for name, value in macros.items():
        assert getattr(_lib, name) == value, name


def test_no_gpu_is_an_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from grilly2_b200 import _lib
    lib = _lib.load()
    out = ctypes.c_void_p()
    assert lib.gq_create(0, ctypes.byref(out)) == _lib.GQ_ERR
    assert "no CUDA device" in _lib.last_error() and not out.value
    import numpy as np
    import grilly2_b200 as g
    with pytest.raises(RuntimeError, match="no CPU path"):
        g.from_numpy(np.zeros(4, dtype=np.float32))


def test_null_context_is_reported_not_crashed():
    from grilly2_b200 import _lib
    lib = _lib.load()
    assert lib.gq_synchronize(None) == _lib.GQ_ERR
    assert "null context" in _lib.last_error()
    out = ctypes.c_uint64()
    assert lib.gq_buffer_create(None, 16, 0, ctypes.byref(out)) == _lib.GQ_ERR


def test_product_does_not_import_the_oracle():
    """The oracle is test infrastructure: nothing under the package may name it."""
    pkg = os.path.join(ROOT, "grilly2_b200")
    for base, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".h", ".cuh")):
                text = open(os.path.join(base, f)).read()
                assert "import oracle" not in text and "from oracle" not in text and "liboracle" not in text, f
