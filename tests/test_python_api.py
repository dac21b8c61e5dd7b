"""Argument validation of the NumPy-facing API; the messages are the ones upstream's tests match
(upstream tests/test_python_api_rows.py:163-306).  No call here reaches the GPU."""
import numpy as np
import pytest

import libgguf_b200 as g
from libgguf_b200 import GGMLQuantizationType as Q


def test_quantize_rejects_bad_width():
    with pytest.raises(ValueError, match=r"quantize row width must be a multiple of this quantization type's block size \(256\)"):
        g.quantize_rows(np.zeros((2, 100), np.float32), Q.Q4_K)
    with pytest.raises(ValueError, match="unsupported quantization type or row width"):
        g.quantize_rows(np.zeros((2, 256), np.float32), Q.Q8_K)


def test_quantize_rejects_bad_imatrix():
    with pytest.raises(ValueError, match="imatrix must be a one-dimensional float32 array"):
        g.quantize_rows(np.zeros((2, 256), np.float32), Q.Q4_K, imatrix=np.ones((2, 256), np.float32))
    with pytest.raises(ValueError, match="imatrix length must match n_per_row"):
        g.quantize_rows(np.zeros((2, 256), np.float32), Q.Q4_K, imatrix=np.ones(128, np.float32))


def test_dequantize_rejects_bad_shapes():
    with pytest.raises(ValueError, match="encoded row width is not a multiple of the quantization block size"):
        g.dequantize_rows(np.zeros((2, 145), np.uint8), Q.Q4_K)
    with pytest.raises(ValueError, match="encoded row width does not match n_per_row"):
        g.dequantize_rows(np.zeros((2, 144), np.uint8), Q.Q4_K, n_per_row=512)
    with pytest.raises(ValueError, match="unsupported quantization type"):
        g.dequantize_rows(np.zeros((2, 4), np.uint8), Q.F32)
    with pytest.raises(ValueError, match="n_per_row must be positive"):
        g.dequantize_rows(np.zeros((2, 144), np.uint8), Q.Q4_K, n_per_row=0)


def test_raw_buffer_checks():
    with pytest.raises(ValueError, match="src buffer size"):
        g.quantize_rows_into_raw(Q.Q8_0, np.zeros(31, np.float32), np.zeros(34, np.uint8), 1, 32)
    with pytest.raises(ValueError, match="dst buffer is too small"):
        g.quantize_rows_into_raw(Q.Q8_0, np.zeros(32, np.float32), np.zeros(33, np.uint8), 1, 32)
    with pytest.raises(ValueError, match="requires an imatrix"):
        g.quantize_rows_into_raw(Q.IQ2_XXS, np.zeros(256, np.float32), np.zeros(66, np.uint8), 1, 256)
    with pytest.raises(ValueError, match="store_rows only supports"):
        g.store_rows(np.zeros((1, 32), np.float32), Q.Q8_0)
    assert g.quantize_rows_into_raw(Q.Q8_0, np.zeros(0, np.float32), np.zeros(0, np.uint8), 0, 32) == 0


def test_c_abi_error_returns_are_zero_without_touching_the_device():
    from libgguf_b200._native import lib
    x = np.zeros(256, np.float32)
    out = np.zeros(1024, np.uint8)
    q = lib.libgguf_quantize_chunk
    assert q(12, x.ctypes.data, out.ctypes.data, 0, 0, 256, None) == 0       # nrows <= 0
    assert q(12, x.ctypes.data, out.ctypes.data, 0, 1, 100, None) == 0       # width not a block multiple
    assert q(12, x.ctypes.data, out.ctypes.data, 128, 1, 256, None) == 0     # start not a row multiple
    assert q(12, x.ctypes.data, out.ctypes.data, -256, 1, 256, None) == 0    # negative start
    assert q(16, x.ctypes.data, out.ctypes.data, 0, 1, 256, None) == 0       # missing required imatrix
    assert q(15, x.ctypes.data, out.ctypes.data, 0, 1, 256, None) == 0       # Q8_K has no row encoder
    d = lib.libgguf_dequantize_chunk
    assert d(12, out.ctypes.data, x.ctypes.data, 0, 0, 256) == 0
    assert d(12, out.ctypes.data, x.ctypes.data, 0, 1, 100) == 0
    assert d(0, out.ctypes.data, x.ctypes.data, 0, 1, 256) == 0              # F32 has no decoder
