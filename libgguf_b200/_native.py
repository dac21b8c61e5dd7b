"""ctypes binding of libgguf_b200.so (the C ABI declared in include/libgguf.h and
include/libgguf_cuda_native.h).

There is no fallback: if the shared library is missing the import raises, and if no CUDA device
is usable the row functions report failure (0 bytes / a non-zero status)."""
from __future__ import annotations

import ctypes
import os
from ctypes import c_bool, c_char_p, c_double, c_float, c_int, c_int32, c_int64, c_size_t, c_uint64, c_void_p, POINTER


class TensorDesc(ctypes.Structure):
    """libgguf_cuda_tensor_desc"""
    _fields_ = [("qtype", c_int64), ("src", c_void_p), ("imatrix", c_void_p), ("dst", c_void_p),
                ("rows", c_int64), ("n_per_row", c_int64)]


class ShardDesc(ctypes.Structure):
    """libgguf_cuda_shard"""
    _fields_ = [("tensor", c_int32), ("row0", c_int64), ("rows", c_int64)]

from pathlib import Path

LIB_PATH = Path(os.environ.get("LIBGGUF_B200_LIBRARY", Path(__file__).with_name("libgguf_b200.so")))

# Every symbol the two public headers declare, with its ctypes signature.
HOST_ABI = {
    "libgguf_row_size": (c_size_t, [c_int, c_int64]),
    "libgguf_type_size": (c_size_t, [c_int]),
    "libgguf_type_name": (c_char_p, [c_int]),
    "libgguf_quantize_requires_imatrix": (c_bool, [c_int]),
    "libgguf_quantize_free": (None, []),
    "libgguf_quantize_chunk": (c_size_t, [c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "libgguf_dequantize_chunk": (c_size_t, [c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64]),
}
NATIVE_ABI = {
    "libgguf_cuda_context_create": (c_int, [c_int, POINTER(c_void_p)]),
    "libgguf_cuda_context_destroy": (None, [c_void_p]),
    "libgguf_cuda_last_error": (c_char_p, [c_void_p]),
    "libgguf_cuda_event_create": (c_int, [c_void_p, POINTER(c_void_p)]),
    "libgguf_cuda_event_destroy": (None, [c_void_p, c_void_p]),
    "libgguf_cuda_event_record": (c_int, [c_void_p, c_void_p]),
    "libgguf_cuda_event_synchronize": (c_int, [c_void_p, c_void_p]),
    "libgguf_cuda_event_elapsed_ms": (c_int, [c_void_p, c_void_p, c_void_p, POINTER(c_float)]),
    "libgguf_cuda_qtype_supported": (c_int, [c_int64]),
    "libgguf_cuda_qtype_needs_imatrix": (c_int, [c_int64]),
    "libgguf_cuda_block_size": (c_int64, [c_int64]),
    "libgguf_cuda_row_size": (c_int64, [c_int64, c_int64]),
    "libgguf_cuda_dequantize_qtype_supported": (c_int, [c_int64]),
    "libgguf_cuda_dequantize_block_size": (c_int64, [c_int64]),
    "libgguf_cuda_dequantize_row_size": (c_int64, [c_int64, c_int64]),
    "libgguf_cuda_buffer_create": (c_int, [c_void_p, c_size_t, POINTER(c_void_p)]),
    "libgguf_cuda_buffer_destroy": (None, [c_void_p, c_void_p]),
    "libgguf_cuda_buffer_resize_discard": (c_int, [c_void_p, c_void_p, c_size_t]),
    "libgguf_cuda_buffer_data": (c_void_p, [c_void_p]),
    "libgguf_cuda_buffer_const_data": (c_void_p, [c_void_p]),
    "libgguf_cuda_buffer_size": (c_size_t, [c_void_p]),
    "libgguf_cuda_host_buffer_create": (c_int, [c_void_p, c_size_t, POINTER(c_void_p)]),
    "libgguf_cuda_host_buffer_destroy": (None, [c_void_p, c_void_p]),
    "libgguf_cuda_host_buffer_resize_discard": (c_int, [c_void_p, c_void_p, c_size_t]),
    "libgguf_cuda_host_buffer_data": (c_void_p, [c_void_p]),
    "libgguf_cuda_host_buffer_const_data": (c_void_p, [c_void_p]),
    "libgguf_cuda_host_buffer_size": (c_size_t, [c_void_p]),
    "libgguf_cuda_h2d": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p, c_size_t]),
    "libgguf_cuda_d2h": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_size_t]),
    "libgguf_cuda_quantize_f32_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64]),
    "libgguf_cuda_dequantize_rows": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "libgguf_cuda_dequantize_rows_on_stream": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "libgguf_cuda_quantize_f32_rows_on_stream": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "libgguf_cuda_thread_last_error": (c_char_p, []),
    "libgguf_cuda_kernel_launch_count": (c_uint64, []),
    "libgguf_cuda_staging_timeouts": (c_int, [c_void_p]),
    "libgguf_cuda_set_staging_wait_limit": (c_int, [c_int]),
    "libgguf_cuda_checked_violations": (c_int, [POINTER(c_uint64)]),
    "libgguf_cuda_host_copy": (None, [c_void_p, c_void_p, c_size_t]),
    "libgguf_cuda_prepare_qtype": (c_int, [c_int64]),
    "libgguf_cuda_quantize_weighted_rows_static": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "libgguf_cuda_quantize_weighted_rows_static_max_rows": (c_int64, []),
    "libgguf_cuda_iq_search_table": (c_int, [c_int64, POINTER(c_int32), POINTER(c_int32), POINTER(c_void_p), POINTER(c_void_p),
                                     POINTER(c_int64), POINTER(c_void_p), POINTER(c_int64)]),
    "libgguf_cuda_iq_scan_records": (c_int, [c_int64, POINTER(c_int32), POINTER(c_void_p), POINTER(c_int64), POINTER(c_void_p),
                                     POINTER(c_int64)]),
    "libgguf_cuda_selftest_fp4": (c_int, [c_float, POINTER(c_uint64)]),
    "libgguf_cuda_selftest_fp4_mode": (c_int, [c_float, c_int, POINTER(c_uint64), POINTER(c_uint64)]),
    "libgguf_cuda_pipeline_create": (c_int, [POINTER(c_int), c_int, c_int, c_size_t, POINTER(c_void_p)]),
    "libgguf_cuda_pipeline_destroy": (None, [c_void_p]),
    "libgguf_cuda_pipeline_last_error": (c_char_p, [c_void_p]),
    "libgguf_cuda_pipeline_quantize": (c_int, [c_void_p, POINTER(TensorDesc), c_int]),
    "libgguf_cuda_pipeline_quantize_typed": (c_int, [c_void_p, POINTER(TensorDesc), POINTER(c_int32), c_int]),
    "libgguf_cuda_pipeline_plan_typed": (c_int64, [POINTER(TensorDesc), POINTER(c_int32), c_int, c_size_t, POINTER(ShardDesc), c_int64]),
    "libgguf_cuda_device_count": (c_int, [POINTER(c_int)]),
    "libgguf_cuda_accumulate_imatrix_on_stream": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "libgguf_cuda_auto_imatrix": (c_int, [c_void_p, c_int64, c_int64, c_void_p]),
    "libgguf_cuda_auto_imatrix_typed": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p]),
    "libgguf_cuda_widen_on_stream": (c_int, [c_void_p, c_int, c_void_p, c_int64, c_void_p]),
    "libgguf_cuda_quantize_rows_from_on_stream": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "libgguf_cuda_pipeline_plan": (c_int64, [POINTER(TensorDesc), c_int, c_size_t, POINTER(ShardDesc), c_int64]),
    "libgguf_cuda_pipeline_stats": (c_int, [c_void_p, POINTER(c_int64), POINTER(c_double), POINTER(c_int64)]),
    "libgguf_cuda_pipeline_inject_failure": (c_int, [c_void_p, c_int, c_int64]),
}


def _load() -> ctypes.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python libgguf_b200/build.py` "
            "(nvcc, sm_100a); libgguf_b200 has no CPU implementation to fall back to")
    lib = ctypes.CDLL(str(LIB_PATH))
    for table in (HOST_ABI, NATIVE_ABI):
        for name, (restype, argtypes) in table.items():
            fn = getattr(lib, name)  # AttributeError if the library does not export the symbol
            fn.restype = restype
            fn.argtypes = argtypes
    return lib


lib = _load()
