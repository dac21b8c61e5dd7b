from __future__ import annotations

from .ops import dequantize, quantize, quantize_weighted

__all__ = ["dequantize", "quantize", "quantize_weighted"]
