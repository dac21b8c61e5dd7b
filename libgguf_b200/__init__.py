"""Row quantize / dequantize for GGUF block formats on NVIDIA B200 (sm_100a).

The functions below keep the names, arguments, return shapes and error messages of upstream's
NumPy-facing API (upstream src/libgguf/__init__.py:26-244) and forward to the C ABI of
libgguf_b200.so, which runs CUDA kernels; host arrays are staged through the GPU.  A missing
shared library is an ImportError and a missing GPU makes the row calls raise RuntimeError:
there is no CPU implementation in this package.
"""
from __future__ import annotations

import atexit
from typing import Any

import numpy as np

from ._metadata import (
    GGML_QUANT_SIZES,
    GGMLQuantizationType,
    QK_K,
    quant_shape_from_byte_shape,
    quant_shape_to_byte_shape,
)
from ._native import lib as _lib


def _qtype_value(qtype: int | Any) -> int:
    return int(getattr(qtype, "value", qtype))


def row_size(qtype: int | Any, n_per_row: int) -> int:
    qtype_value = _qtype_value(qtype)
    n = int(n_per_row)
    if n <= 0:
        return 0
    block_size = _BLOCK_SIZES.get(qtype_value)
    if block_size is not None and block_size > 1 and n % block_size != 0:
        return 0
    return int(_lib.libgguf_row_size(qtype_value, n))


def type_size(qtype: int | Any) -> int:
    return int(_lib.libgguf_type_size(_qtype_value(qtype)))


def type_name(qtype: int | Any) -> str:
    return _lib.libgguf_type_name(_qtype_value(qtype)).decode()


def quantize_requires_imatrix(qtype: int | Any) -> bool:
    return bool(_lib.libgguf_quantize_requires_imatrix(_qtype_value(qtype)))


_BLOCK_SIZES: dict[int, int] = {int(q): bs for q, (bs, _) in GGML_QUANT_SIZES.items()}
_STORAGE_QTYPE_DTYPES: dict[int, np.dtype] = {0: np.dtype(np.float32), 1: np.dtype(np.float16)}
_STORAGE_QTYPES = frozenset((*_STORAGE_QTYPE_DTYPES, 30))
_SUPPORTED_ROW_QTYPES = frozenset(q for q, bs in _BLOCK_SIZES.items() if row_size(q, bs) > 0)
_SUPPORTED_QUANTIZED_QTYPES = frozenset(q for q in _SUPPORTED_ROW_QTYPES if q not in _STORAGE_QTYPES)


def _validated_row_size(qtype_value: int, n_per_row: int, operation: str) -> int:
    if n_per_row <= 0:
        raise ValueError("n_per_row must be positive")
    if operation == "dequantize" and qtype_value not in _SUPPORTED_QUANTIZED_QTYPES:
        raise ValueError("unsupported quantization type or row width")
    bytes_per_row = row_size(qtype_value, n_per_row)
    if bytes_per_row > 0:
        return bytes_per_row
    block_size = _BLOCK_SIZES.get(qtype_value)
    if block_size is not None and block_size > 1 and n_per_row % block_size != 0:
        raise ValueError(
            f"{operation} row width must be a multiple of this quantization type's block size ({block_size})")
    raise ValueError("unsupported quantization type or row width")


def _validate_imatrix(imatrix: Any, n_per_row: int) -> np.ndarray:
    quant_weights = np.ascontiguousarray(imatrix, dtype=np.float32)
    if quant_weights.ndim != 1:
        raise ValueError("imatrix must be a one-dimensional float32 array")
    if quant_weights.shape[0] != n_per_row:
        raise ValueError("imatrix length must match n_per_row")
    return quant_weights


def _readable(buf: Any, name: str) -> np.ndarray:
    try:
        arr = np.frombuffer(buf, dtype=np.uint8) if not isinstance(buf, np.ndarray) else buf
    except (TypeError, ValueError) as exc:
        raise ValueError(f"{name} must support the buffer protocol") from exc
    if isinstance(arr, np.ndarray) and not arr.flags.c_contiguous:
        raise ValueError(f"{name} must be C-contiguous")
    return arr


def quantize_rows_into_raw(qtype: int | Any, src: Any, dst: Any, n_rows: int, n_per_row: int,
                           imatrix: Any | None = None) -> int:
    """Quantizes n_rows x n_per_row float32 values from `src` into the writable buffer `dst`.
    Returns the number of bytes written (upstream csrc/_libgguf_module.cpp:1757-1912)."""
    qtype_value = _qtype_value(qtype)
    n_rows, n_per_row = int(n_rows), int(n_per_row)
    bytes_per_row = _validated_row_size(qtype_value, n_per_row, "quantize")
    if n_rows < 0:
        raise ValueError("n_rows must be non-negative")
    src_arr = _readable(src, "src")
    dst_arr = _readable(dst, "dst")
    if src_arr.nbytes != n_rows * n_per_row * 4:
        raise ValueError("src buffer size does not match n_rows * n_per_row float32 values")
    if dst_arr.nbytes < n_rows * bytes_per_row:
        raise ValueError("dst buffer is too small for the quantized rows")
    if isinstance(dst_arr, np.ndarray) and not dst_arr.flags.writeable:
        raise ValueError("dst must be writable")
    weights = None
    if imatrix is not None:
        weights = _validate_imatrix(imatrix, n_per_row)
    elif quantize_requires_imatrix(qtype_value):
        raise ValueError("this quantization type requires an imatrix")
    if n_rows == 0:
        return 0
    written = int(_lib.libgguf_quantize_chunk(
        qtype_value, src_arr.ctypes.data, dst_arr.ctypes.data, 0, n_rows, n_per_row,
        weights.ctypes.data if weights is not None else None))
    if written != n_rows * bytes_per_row:
        raise RuntimeError(
            f"libgguf_quantize_chunk wrote {written} bytes, expected {n_rows * bytes_per_row} "
            "(no usable CUDA device, or the device call failed)")
    return written


def quantize_rows_raw(qtype: int | Any, src: Any, n_rows: int, n_per_row: int, imatrix: Any | None = None) -> bytes:
    qtype_value = _qtype_value(qtype)
    bytes_per_row = _validated_row_size(qtype_value, int(n_per_row), "quantize")
    out = np.empty(int(n_rows) * bytes_per_row, dtype=np.uint8)
    quantize_rows_into_raw(qtype_value, src, out, n_rows, n_per_row, imatrix)
    return out.tobytes()


def dequantize_rows_into_raw(qtype: int | Any, src: Any, dst: Any, n_rows: int, n_per_row: int) -> int:
    """Decodes n_rows encoded rows from `src` into float32 values in the writable buffer `dst`.
    Returns the number of bytes written (upstream csrc/_libgguf_module.cpp:2008-2105)."""
    qtype_value = _qtype_value(qtype)
    n_rows, n_per_row = int(n_rows), int(n_per_row)
    bytes_per_row = _validated_row_size(qtype_value, n_per_row, "dequantize")
    if n_rows < 0:
        raise ValueError("n_rows must be non-negative")
    src_arr = _readable(src, "src")
    dst_arr = _readable(dst, "dst")
    if src_arr.nbytes != n_rows * bytes_per_row:
        raise ValueError("src buffer size does not match n_rows encoded rows")
    if dst_arr.nbytes < n_rows * n_per_row * 4:
        raise ValueError("dst buffer is too small for the dequantized rows")
    if isinstance(dst_arr, np.ndarray) and not dst_arr.flags.writeable:
        raise ValueError("dst must be writable")
    if n_rows == 0:
        return 0
    written = int(_lib.libgguf_dequantize_chunk(qtype_value, src_arr.ctypes.data, dst_arr.ctypes.data, 0, n_rows, n_per_row))
    if written != n_rows * n_per_row * 4:
        raise RuntimeError(
            f"libgguf_dequantize_chunk wrote {written} bytes, expected {n_rows * n_per_row * 4} "
            "(no usable CUDA device, or the device call failed)")
    return written


def dequantize_rows_raw(qtype: int | Any, src: Any, n_rows: int, n_per_row: int) -> bytes:
    out = np.empty(int(n_rows) * int(n_per_row), dtype=np.float32)
    dequantize_rows_into_raw(qtype, src, out, n_rows, n_per_row)
    return out.tobytes()


def auto_imatrix(rows: np.ndarray) -> np.ndarray:
    """Column sums of squares of a 2-D fp32 matrix, added in row order on the GPU: the importance weights upstream
    derives from the data when a type needs them and none are given (upstream __init__.py:186-189, same bits as
    np.sum(rows * rows, axis=0, dtype=np.float32))."""
    rows = np.ascontiguousarray(rows, dtype=np.float32)
    if rows.ndim != 2:
        raise ValueError("auto_imatrix expects a two-dimensional array")
    out = np.zeros(rows.shape[1], dtype=np.float32)
    if rows.shape[1] == 0:
        return out
    status = _lib.libgguf_cuda_auto_imatrix(rows.ctypes.data, rows.shape[0], rows.shape[1], out.ctypes.data)
    if status != 0:
        raise RuntimeError(f"libgguf_cuda_auto_imatrix failed with status {status}")
    return out


def quantize_rows(data: np.ndarray, qtype: int | Any, imatrix: Any | None = None) -> np.ndarray:
    """fp32 array [..., n] -> uint8 array [..., bytes_per_row] (upstream __init__.py:171-196).
    Types that require importance weights get the column sums of squares when none are given."""
    qtype_value = _qtype_value(qtype)
    if qtype_value in _STORAGE_QTYPES:
        return store_rows(data, qtype_value)
    rows = np.ascontiguousarray(data, dtype=np.float32)
    if rows.ndim == 0:
        raise ValueError("Expected an array with at least one dimension")
    n_rows = int(np.prod(rows.shape[:-1], dtype=np.int64)) if rows.ndim > 1 else 1
    n_per_row = int(rows.shape[-1])
    if imatrix is not None:
        quant_weights = _validate_imatrix(imatrix, n_per_row)
    elif quantize_requires_imatrix(qtype_value):
        quant_weights = auto_imatrix(rows.reshape((-1, n_per_row)))
    else:
        quant_weights = None
    bytes_per_row = _validated_row_size(qtype_value, n_per_row, "quantize")
    out = np.empty((*rows.shape[:-1], bytes_per_row), dtype=np.uint8)
    quantize_rows_into_raw(qtype_value, rows, out, n_rows, n_per_row, quant_weights)
    return out


def store_rows(data: np.ndarray, qtype: int | Any) -> np.ndarray:
    """F32 / F16 / BF16 storage of fp32 rows (upstream __init__.py:199-217)."""
    rows = np.ascontiguousarray(data, dtype=np.float32)
    if rows.ndim == 0:
        raise ValueError("Expected an array with at least one dimension")
    qtype_value = _qtype_value(qtype)
    if qtype_value not in _STORAGE_QTYPES:
        raise ValueError("store_rows only supports F32, F16, and BF16 storage types")
    n_rows = int(np.prod(rows.shape[:-1], dtype=np.int64)) if rows.ndim > 1 else 1
    n_per_row = int(rows.shape[-1])
    bytes_per_row = _validated_row_size(qtype_value, n_per_row, "store")
    out = np.empty((*rows.shape[:-1], bytes_per_row), dtype=np.uint8)
    quantize_rows_into_raw(qtype_value, rows, out, n_rows, n_per_row)
    dtype = _STORAGE_QTYPE_DTYPES.get(qtype_value)
    if dtype is None:
        return out
    return out.view(dtype).reshape(rows.shape)


def dequantize_rows(data: Any, qtype: int | Any, n_per_row: int | None = None) -> np.ndarray:
    """uint8 array [..., bytes_per_row] -> fp32 array [..., n] (upstream __init__.py:220-244)."""
    rows = np.ascontiguousarray(data, dtype=np.uint8)
    if rows.ndim == 0:
        raise ValueError("Expected an array with at least one dimension")
    qtype_value = _qtype_value(qtype)
    bytes_per_row = int(rows.shape[-1])
    if n_per_row is None:
        if qtype_value not in _SUPPORTED_QUANTIZED_QTYPES:
            raise ValueError("unsupported quantization type")
        block_size = _BLOCK_SIZES[qtype_value]
        block_bytes = type_size(qtype_value)
        if bytes_per_row % block_bytes != 0:
            raise ValueError("encoded row width is not a multiple of the quantization block size")
        n_per_row = bytes_per_row // block_bytes * block_size
    else:
        n_per_row = int(n_per_row)
    if _validated_row_size(qtype_value, n_per_row, "dequantize") != bytes_per_row:
        raise ValueError("encoded row width does not match n_per_row for this quantization type")
    n_rows = int(np.prod(rows.shape[:-1], dtype=np.int64)) if rows.ndim > 1 else 1
    out = np.empty((*rows.shape[:-1], n_per_row), dtype=np.float32)
    dequantize_rows_into_raw(qtype_value, rows, out, n_rows, n_per_row)
    return out


atexit.register(_lib.libgguf_quantize_free)

__all__ = [
    "GGMLQuantizationType", "GGML_QUANT_SIZES", "QK_K",
    "dequantize_rows", "dequantize_rows_into_raw", "dequantize_rows_raw",
    "auto_imatrix", "quantize_requires_imatrix", "quantize_rows", "quantize_rows_into_raw", "quantize_rows_raw",
    "quant_shape_from_byte_shape", "quant_shape_to_byte_shape",
    "row_size", "store_rows", "type_name", "type_size",
]
