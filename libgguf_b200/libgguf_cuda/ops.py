"""Torch ops `_C_gguf::quantize` / `_C_gguf::dequantize` and their Python entry points.

The two operators are registered under upstream's names and schemas (upstream
src/libgguf/libgguf_cuda/csrc/torch_bindings.cpp:12-20), CUDA dispatch key only, with the same
argument checks and messages as upstream's TORCH_CHECKs (csrc/cuda_quantize.cu:11-51,
csrc/cuda_dequantize.cu:37-69), and with fake / meta implementations that follow upstream's
(src/libgguf/libgguf_cuda/ops.py:17-164), so `torch.ops._C_gguf.*`, FakeTensorMode, the meta
device, torch.compile and torch.export see what they see with upstream's extension.  PyTorch
is used for exactly three things in the CUDA implementations: allocating the output tensor,
naming the device, and handing over the current stream; the work is done by libgguf_b200.so
through its device-pointer C ABI.

`quantize` behaves like upstream's op: the importance weights are read only by the types that
cannot be quantized without them.  `quantize_weighted` (an addition, `_C_gguf::quantize_weighted`)
hands the weights to every type whose CPU quantizer honours them, which is what
libgguf.quantize_rows(data, qtype, imatrix) computes on the CPU.  The output element count is
not limited to int32 (upstream: m * n <= INT_MAX).
"""
from __future__ import annotations

import torch

from .. import GGMLQuantizationType, GGML_QUANT_SIZES, quantize_requires_imatrix
from .._native import lib as _lib

_OUT_DTYPES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
_DEVICE_TYPES = ("cuda", "meta")


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


def _check_quantize(W: torch.Tensor, quant_type: int, imatrix, use_imatrix: bool, real: bool) -> tuple[int, int, int]:
    """Shared by the CUDA and the fake implementation; returns (rows, n, row_size).  `real` adds the checks that
    only make sense for tensors with storage."""
    if W.device.type not in _DEVICE_TYPES:
        raise RuntimeError("CUDA quantize expects a CUDA tensor")
    if W.dtype != torch.float32:
        raise RuntimeError("CUDA quantize expects float32 input")
    if W.dim() < 1:
        raise RuntimeError("CUDA quantize expects at least one dimension")
    if real and not W.is_contiguous():
        raise RuntimeError("CUDA quantize expects contiguous input")
    block, type_size = _quant_geometry(quant_type, "quantize")
    n = W.shape[-1]
    if n % block != 0:
        raise RuntimeError("CUDA quantize input width must be divisible by the quantization block size")
    if imatrix is None and quantize_requires_imatrix(quant_type):
        raise RuntimeError(f"CUDA quantize requires imatrix for GGML quantization type: {quant_type}")
    if use_imatrix and imatrix is not None:
        if imatrix.device.type not in _DEVICE_TYPES:
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
    m = 1
    for s in W.shape[:-1]:
        m *= s
    return m, n, n // block * type_size


def _check_dequantize(W: torch.Tensor, quant_type: int, m, n, dtype, real: bool) -> torch.dtype:
    if W.device.type not in _DEVICE_TYPES:
        raise RuntimeError("CUDA dequantize expects a CUDA tensor")
    if W.dtype != torch.uint8:
        raise RuntimeError("CUDA dequantize expects uint8 input")
    if real and not W.is_contiguous():
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
    return dtype_


# ---- CUDA implementations ----------------------------------------------------------------------
def _quantize_cuda_impl(W: torch.Tensor, quant_type: int, imatrix, use_imatrix: bool) -> torch.Tensor:
    m, n, row_size = _check_quantize(W, quant_type, imatrix, use_imatrix, real=True)
    out = torch.empty((*W.shape[:-1], row_size), dtype=torch.uint8, device=W.device)
    if m * n == 0:
        return out
    imatrix_ptr = imatrix.data_ptr() if (use_imatrix and imatrix is not None) else None
    with torch.cuda.device(W.device):
        stream = torch.cuda.current_stream(W.device).cuda_stream
        _status(_lib.libgguf_cuda_quantize_f32_rows_on_stream(W.data_ptr(), imatrix_ptr, out.data_ptr(), int(quant_type),
                                                              m, n, stream), "quantize")
    return out


def _quantize_cuda(W: torch.Tensor, type: int, imatrix: torch.Tensor | None = None) -> torch.Tensor:
    # upstream reads the weights only when the type cannot do without them (cuda_quantize.cu:37-49)
    return _quantize_cuda_impl(W, type, imatrix, bool(quantize_requires_imatrix(type)) if _known(type) else False)


def _quantize_weighted_cuda(W: torch.Tensor, type: int, imatrix: torch.Tensor) -> torch.Tensor:
    return _quantize_cuda_impl(W, type, imatrix, True)


def _dequantize_cuda(W: torch.Tensor, type: int, m: int, n: int, dtype: torch.dtype | None = None) -> torch.Tensor:
    dtype_ = _check_dequantize(W, type, m, n, dtype, real=True)
    out = torch.empty((m, n), dtype=dtype_, device=W.device)
    with torch.cuda.device(W.device):
        stream = torch.cuda.current_stream(W.device).cuda_stream
        _status(_lib.libgguf_cuda_dequantize_rows_on_stream(W.data_ptr(), int(type), m, n, _OUT_DTYPES[dtype_],
                                                            out.data_ptr(), stream), "dequantize")
    return out


def _known(quant_type: int) -> bool:
    try:
        GGMLQuantizationType(int(quant_type))
        return True
    except ValueError:
        return False


# ---- fake / meta implementations (shape, dtype and argument validation only) -------------------------------
def _quantize_fake(W: torch.Tensor, type: int, imatrix: torch.Tensor | None = None) -> torch.Tensor:
    use = bool(quantize_requires_imatrix(type)) if _known(type) else False
    _, _, row_size = _check_quantize(W, type, imatrix, use, real=False)
    return torch.empty((*W.shape[:-1], row_size), dtype=torch.uint8, device=W.device)


def _quantize_weighted_fake(W: torch.Tensor, type: int, imatrix: torch.Tensor) -> torch.Tensor:
    _, _, row_size = _check_quantize(W, type, imatrix, True, real=False)
    return torch.empty((*W.shape[:-1], row_size), dtype=torch.uint8, device=W.device)


def _dequantize_fake(W: torch.Tensor, type: int, m, n, dtype: torch.dtype | None = None) -> torch.Tensor:
    dtype_ = _check_dequantize(W, type, m, n, dtype, real=False)
    return torch.empty((m, n), dtype=dtype_, device=W.device)


# ---- registration (once per process; upstream does this from its C++ extension) ------------------
def _register() -> "torch.library.Library | None":
    if hasattr(torch.ops, "_C_gguf") and hasattr(torch.ops._C_gguf, "dequantize"):
        return None  # another copy of this module (or upstream's extension) already defined the operators
    try:
        from torch.library import register_fake
    except ImportError:  # older torch
        from torch.library import impl_abstract as register_fake
    library = torch.library.Library("_C_gguf", "DEF")
    library.define("dequantize(Tensor W, int type, SymInt m, SymInt n, ScalarType? dtype) -> Tensor")
    library.define("quantize(Tensor W, int type, Tensor? imatrix=None) -> Tensor")
    library.define("quantize_weighted(Tensor W, int type, Tensor imatrix) -> Tensor")
    library.impl("dequantize", _dequantize_cuda, "CUDA")
    library.impl("quantize", _quantize_cuda, "CUDA")
    library.impl("quantize_weighted", _quantize_weighted_cuda, "CUDA")
    register_fake("_C_gguf::dequantize")(_dequantize_fake)
    register_fake("_C_gguf::quantize")(_quantize_fake)
    register_fake("_C_gguf::quantize_weighted")(_quantize_weighted_fake)
    return library


_LIBRARY = _register()  # kept alive: dropping the Library object would unregister the operators


def _reject_cpu(W: torch.Tensor, what: str) -> None:
    # The operators have no CPU kernel; say so in upstream's words instead of the dispatcher's.
    if W.device.type == "cpu" and type(W) is torch.Tensor:
        raise RuntimeError(f"CUDA {what} expects a CUDA tensor")


def quantize(W: torch.Tensor, quant_type: int, imatrix: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 CUDA tensor [..., n] -> uint8 CUDA tensor [..., row_size], on the current stream (upstream ops.py:173-176)."""
    _reject_cpu(W, "quantize")
    return torch.ops._C_gguf.quantize(W, quant_type, imatrix)


def quantize_weighted(W: torch.Tensor, quant_type: int, imatrix: torch.Tensor) -> torch.Tensor:
    """As `quantize`, with the importance weights applied by every type whose quantizer has a weighted form
    (the K-quants, Q4_0 ... Q5_1, IQ4 and all lattice types); no upstream counterpart among the Torch ops."""
    _reject_cpu(W, "quantize")
    return torch.ops._C_gguf.quantize_weighted(W, quant_type, imatrix)


def dequantize(W: torch.Tensor, quant_type: int, m: int, n: int, dtype: torch.dtype | None = None) -> torch.Tensor:
    """uint8 CUDA tensor holding m encoded rows -> [m, n] tensor of `dtype` (default float16) (upstream ops.py:167-170)."""
    _reject_cpu(W, "dequantize")
    return torch.ops._C_gguf.dequantize(W, quant_type, m, n, dtype)
