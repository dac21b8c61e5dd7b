"""Torch entry points `quantize` / `dequantize` over CUDA tensors.

Same call signatures, argument checks and error messages as upstream's Torch ops
(upstream src/libgguf/libgguf_cuda/ops.py:167-176 and the TORCH_CHECKs of
csrc/cuda_quantize.cu:11-51, csrc/cuda_dequantize.cu:37-69).  PyTorch is used for exactly three
things here: allocating the output tensor, naming the device, and handing over the current
stream; the work is done by libgguf_b200.so through its device-pointer C ABI.

Differences from upstream, both additive: `imatrix` is honoured whenever it is given (upstream
forwards it only for the types that require it), and the output element count is not limited to
int32.
"""
from __future__ import annotations

import torch

from .. import GGMLQuantizationType, GGML_QUANT_SIZES, quantize_requires_imatrix
from .._native import lib as _lib

_OUT_DTYPES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def _quant_geometry(quant_type: int, what: str) -> tuple[int, int]:
    try:
        qtype = GGMLQuantizationType(int(quant_type))
    except ValueError:
        raise RuntimeError(f"Unsupported GGML quantization type for CUDA {what}: {quant_type}") from None
    if what == "quantize":
        supported = bool(_lib.libgguf_cuda_qtype_supported(int(qtype)))
    else:
        supported = bool(_lib.libgguf_cuda_dequantize_qtype_supported(int(qtype)))
    if not supported:
        raise RuntimeError(f"Unsupported GGML quantization type for CUDA {what}: {quant_type}")
    return GGML_QUANT_SIZES[qtype]


def _status(status: int, what: str) -> None:
    if status != 0:
        raise RuntimeError(f"CUDA {what} failed: {_lib.libgguf_cuda_thread_last_error().decode()} (status {status})")


def quantize(W: torch.Tensor, quant_type: int, imatrix: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 CUDA tensor [..., n] -> uint8 CUDA tensor [..., row_size], on the current stream."""
    if not W.is_cuda:
        raise RuntimeError("CUDA quantize expects a CUDA tensor")
    if W.dtype != torch.float32:
        raise RuntimeError("CUDA quantize expects float32 input")
    if W.dim() < 1:
        raise RuntimeError("CUDA quantize expects at least one dimension")
    if not W.is_contiguous():
        raise RuntimeError("CUDA quantize expects contiguous input")
    block, type_size = _quant_geometry(quant_type, "quantize")
    n = W.shape[-1]
    if n % block != 0:
        raise RuntimeError("CUDA quantize input width must be divisible by the quantization block size")
    row_size = n // block * type_size
    m = 1
    for s in W.shape[:-1]:
        m *= s
    imatrix_ptr = None
    if imatrix is None and quantize_requires_imatrix(quant_type):
        raise RuntimeError(f"CUDA quantize requires imatrix for GGML quantization type: {quant_type}")
    if imatrix is not None:
        if not imatrix.is_cuda:
            raise RuntimeError("CUDA quantize imatrix must be a CUDA tensor")
        if imatrix.device != W.device:
            raise RuntimeError("CUDA quantize imatrix must be on the same device as input")
        if imatrix.dtype != torch.float32:
            raise RuntimeError("CUDA quantize imatrix must be float32")
        if imatrix.dim() != 1:
            raise RuntimeError("CUDA quantize imatrix must be one-dimensional")
        if imatrix.numel() < n:
            raise RuntimeError("CUDA quantize imatrix must have at least input width elements")
        if not imatrix.is_contiguous():
            raise RuntimeError("CUDA quantize imatrix must be contiguous")
        imatrix_ptr = imatrix.data_ptr()
    out = torch.empty((*W.shape[:-1], row_size), dtype=torch.uint8, device=W.device)
    if m * n == 0:
        return out
    with torch.cuda.device(W.device):
        stream = torch.cuda.current_stream(W.device).cuda_stream
        _status(_lib.libgguf_cuda_quantize_f32_rows_on_stream(W.data_ptr(), imatrix_ptr, out.data_ptr(), int(quant_type),
                                                              m, n, stream), "quantize")
    return out


def dequantize(W: torch.Tensor, quant_type: int, m: int, n: int, dtype: torch.dtype | None = None) -> torch.Tensor:
    """uint8 CUDA tensor holding m encoded rows -> [m, n] tensor of `dtype` (default float16)."""
    if not W.is_cuda:
        raise RuntimeError("CUDA dequantize expects a CUDA tensor")
    if W.dtype != torch.uint8:
        raise RuntimeError("CUDA dequantize expects uint8 input")
    if not W.is_contiguous():
        raise RuntimeError("CUDA dequantize expects contiguous input")
    if m <= 0:
        raise RuntimeError("CUDA dequantize expects positive row count")
    if n <= 0:
        raise RuntimeError("CUDA dequantize expects positive row width")
    dtype_ = dtype or torch.float16
    if dtype_ not in _OUT_DTYPES:
        raise RuntimeError("CUDA dequantize output dtype must be float16, bfloat16, or float32")
    block, type_size = _quant_geometry(quant_type, "dequantize")
    if n % block != 0:
        raise RuntimeError("CUDA dequantize output width must be divisible by the quantization block size")
    expected = m * (n // block * type_size)
    if W.numel() != expected:
        raise RuntimeError(f"CUDA dequantize input has {W.numel()} bytes, expected {expected}")
    out = torch.empty((m, n), dtype=dtype_, device=W.device)
    with torch.cuda.device(W.device):
        stream = torch.cuda.current_stream(W.device).cuda_stream
        _status(_lib.libgguf_cuda_dequantize_rows_on_stream(W.data_ptr(), int(quant_type), m, n, _OUT_DTYPES[dtype_],
                                                            out.data_ptr(), stream), "dequantize")
    return out
