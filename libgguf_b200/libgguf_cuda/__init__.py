from __future__ import annotations

from .ops import dequantize, quantize

__all__ = ["dequantize", "quantize"]
