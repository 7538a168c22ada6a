"""ctypes binding of libgq.so (include/gq.h). This is the only place Python
touches the C ABI; it plays the part the reference's ``grilly-sys`` crate
plays for Rust (crates/grilly-sys/src/lib.rs:63-137: one ``extern "C"`` block
plus a ``check`` that turns GC_ERR into an error value).

There is no fallback: if the library is missing it is built with nvcc, and if
that is impossible, or no B200 is visible, the first use raises.
"""
from __future__ import annotations

import ctypes
import os

from . import build as _build

GQ_OK, GQ_ERR = 0, 1
MEM_DEVICE, MEM_PERSISTENT = 0, 3
KERNEL_AUTO, KERNEL_GEMV, KERNEL_TENSOR, KERNEL_DP4A, KERNEL_IMMA, KERNEL_UMMA, KERNEL_RING = 0, 1, 2, 3, 4, 5, 6
KERNEL_TENSOR_I8 = 7
KERNEL_UMMA_LANES = 8

u64, i32, u32, vp = ctypes.c_uint64, ctypes.c_int32, ctypes.c_uint32, ctypes.c_void_p
P = ctypes.POINTER


class Caps(ctypes.Structure):
    _fields_ = [("device_name", ctypes.c_char * 256), ("cc_major", u32), ("cc_minor", u32), ("sm_count", u32),
                ("max_shared_per_block", u32), ("total_memory", u64), ("l2_bytes", u64)]


class Stats(ctypes.Structure):
    _fields_ = [(n, u64) for n in (
        "launches", "graph_launches", "graph_nodes_replayed", "captures", "syncs", "wait_ns_total", "wait_ns_last",
        "buffer_allocations", "buffers_outstanding", "pool_reuses", "persistent_buffers", "persistent_bytes",
        "persistent_peak", "uploads", "downloads")]


class DecodeLayer(ctypes.Structure):
    _fields_ = [(n, u64) for n in ("input_norm", "qkv_q", "qkv_scale", "qkv_bias", "o_q", "o_scale", "post_norm", "gate_up_q",
                                   "gate_up_scale", "down_q", "down_scale")]


class DecodeDesc(ctypes.Structure):
    _fields_ = ([(n, u64) for n in ("hidden", "heads", "kv_heads", "dim", "inter", "vocab", "layers", "max_len")] +
                [("eps", ctypes.c_float), ("attn_scale", ctypes.c_float)] +
                [(n, u64) for n in ("embed", "final_norm", "head_q", "head_scale", "cos", "sin", "kcache", "vcache", "lens")] +
                [("layer", P(DecodeLayer))])


# name -> argument types; every function but the three noted returns int32 status
PROTOTYPES = {
    "gq_create": [i32, P(vp)],
    "gq_caps_get": [vp, P(Caps)],
    "gq_buffer_create": [vp, u64, u32, P(u64)],
    "gq_buffer_release": [vp, u64],
    "gq_buffer_size": [vp, u64, P(u64)],
    "gq_buffer_wrap": [vp, vp, u64, P(u64)],
    "gq_buffer_ptr": [vp, u64, P(vp)],
    "gq_stream": [vp, P(vp)],
    "gq_upload": [vp, u64, u64, vp, u64],
    "gq_download": [vp, u64, u64, vp, u64],
    "gq_upload_async": [vp, u64, u64, vp, u64],
    "gq_download_async": [vp, u64, u64, vp, u64],
    "gq_host_alloc": [vp, u64, P(vp)],
    "gq_host_free": [vp, vp],
    "gq_copy": [vp, u64, u64, u64, u64, u64],
    "gq_fill": [vp, u64, u64, u64, u32],
    "gq_synchronize": [vp],
    "gq_stats_get": [vp, P(Stats)],
    "gq_persistent_peak_reset": [vp],
    "gq_int8_quantize": [vp, u64, u64, u64, u64, u64, u64],
    "gq_int8_quantize_rows": [vp, u64, u64, u64, u64, u64, u64, u64, u64],
    "gq_int4_quantize_rows": [vp, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64],
    "gq_int8_linear": [vp, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, i32],
    "gq_int8_dequantize": [vp, u64, u64, u64, u64, u64],
    "gq_int4_quantize": [vp, u64, u64, u64, u64, u64, u64, u64, u64],
    "gq_int4_linear": [vp, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, i32],
    "gq_int4_dequantize": [vp, u64, u64, u64, u64, u64, u64, u64],
    "gq_gptq_hessian_add": [vp, u64, u64, u64, u64, u64],
    "gq_gptq_quantize": [vp, u64, u64, u64, u64, u64, u64, u64, u64, u64],
    "gq_begin_capture": [vp],
    "gq_end_capture": [vp, P(vp)],
    "gq_capturing": [vp, P(u32)],
    "gq_graph_replay": [vp, vp],
    "gq_graph_nodes": [vp, P(u64)],
    "gq_embedding": [vp, u64, u64, u64, u64, u64, u64],
    "gq_add_rms_norm": [vp, u64, u64, u64, u64, u64, ctypes.c_float, u64, u64],
    "gq_rope_kv_append": [vp, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64],
    "gq_kv_advance": [vp, u64, u64, u64],
    "gq_attn_scratch_bytes": [vp, u64, u64, u64, P(u64)],
    "gq_attn_decode": [vp, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, ctypes.c_float, u64, u64],
    "gq_attn_decode_static": [vp, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, ctypes.c_float, u64],
    "gq_attn_decode_rope": [vp, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, ctypes.c_float, u64, u64],
    "gq_int8_linear_norm": [vp, u64, u64, u64, ctypes.c_float, u64, u64, u64, u64, u64, u64, u64, u64],
    "gq_int8_linear_swiglu": [vp, u64, u64, u64, u64, u64, u64, u64, u64],
    "gq_attn_prefill": [vp, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, ctypes.c_float, u64, u64],
    "gq_kv_advance_by": [vp, u64, u64, u64, u64],
    "gq_swiglu": [vp, u64, u64, u64, u64],
    "gq_argmax_rows": [vp, u64, u64, u64, u64],
    "gq_decode_plan_create": [vp, P(DecodeDesc), P(vp)],
    "gq_decode_plan_step": [vp, vp, u64, u64, u64],
    "gq_sample": [vp, u64, u64, u64, u64, u64, u64, u32, u32, ctypes.c_double, u64, ctypes.c_double, ctypes.c_double, u64, u64, u64, u64, u64, u64],
    "gq_comm_unique_id": [vp, u64],
    "gq_comm_create": [vp, i32, i32, vp, P(vp)],
    "gq_all_gather_columns": [vp, vp, u64, u64, u64, u64],
    "gq_buffer_ipc_export": [vp, u64, vp, u64],
    "gq_buffer_ipc_open": [vp, vp, u64, P(u64)],
    "gq_peer_gather": [vp, u64, u64, u64, i32, i32, P(u64), u64, u64],
    "gq_int4_linear_gather": [vp, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, i32, i32, P(u64), u64, u64],
    "gq_set_wait_limit_us": [vp, u64],
    "gq_int8_linear_backward": [vp, u64, u64, u64, u64, u64, u64, u64, u64, u64],
    "gq_int4_linear_backward": [vp, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64, u64],
}
VOID_FUNCTIONS = {"gq_destroy": [vp], "gq_graph_destroy": [vp, vp], "gq_comm_destroy": [vp, vp], "gq_decode_plan_destroy": [vp, vp]}

_lib = None


def library_path() -> str:
    return _build.OUT


def load() -> ctypes.CDLL:
    """The loaded library, building it first if the binary is missing."""
    global _lib
    if _lib is None:
        path = _build.OUT
        if not os.path.exists(path):
            path = _build.build()
        lib = ctypes.CDLL(path)
        for name, args in PROTOTYPES.items():
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = args, i32
        for name, args in VOID_FUNCTIONS.items():
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = args, None
        lib.gq_last_error.argtypes, lib.gq_last_error.restype = [], ctypes.c_char_p
        _lib = lib
    return _lib


def last_error() -> str:
    return load().gq_last_error().decode("utf-8", "replace")


def check(status: int) -> None:
    """GQ_ERR -> a Python exception, as the reference's binding maps its core
    errors (crates/grilly-py/src/lib.rs:36-46): RuntimeError for everything the
    C side reports."""
    if status != GQ_OK:
        raise RuntimeError(last_error())
