"""Load-time decoding of GGUF tensors: stored bytes -> pinned staging -> GPU -> dequantize kernel -> torch tensor.

The counterpart of reading a tensor with upstream's GGUFFile.read_tensor_bytes (src/libgguf/inspect.py:113-216) and
passing it to libgguf_cuda.dequantize: nothing is decoded on the CPU, the encoded bytes are what crosses the host link.
"""
from __future__ import annotations

import numpy as np
import torch

from .. import GGML_QUANT_SIZES, GGMLQuantizationType
from ..gguf_file import GGUFFile
from . import ops

_STORAGE = {int(GGMLQuantizationType.F32): torch.float32, int(GGMLQuantizationType.F16): torch.float16,
            int(GGMLQuantizationType.BF16): torch.bfloat16}


def load_tensor(gguf: GGUFFile, name: str, device="cuda", dtype: torch.dtype = torch.float16, stream=None) -> torch.Tensor:
    """The named tensor in its original shape (outermost dimension first) as `dtype` on `device`."""
    info = gguf.tensors[name]
    raw = gguf.tensor_bytes(name)
    staged = torch.empty(info.nbytes, dtype=torch.uint8).pin_memory()
    staged.numpy()[:] = raw
    dev = torch.device(device)
    with torch.cuda.device(dev), torch.cuda.stream(stream or torch.cuda.current_stream(dev)):
        on_gpu = staged.to(dev, non_blocking=True)
        if info.qtype in _STORAGE:
            out = on_gpu.view(_STORAGE[info.qtype]).reshape(info.shape).to(dtype)
        else:
            n = info.shape[-1]
            rows = int(np.prod(info.shape[:-1], dtype=np.int64)) if len(info.shape) > 1 else 1
            block, type_size = GGML_QUANT_SIZES[GGMLQuantizationType(info.qtype)]
            out = ops.dequantize(on_gpu.view(rows, n // block * type_size), info.qtype, rows, n, dtype).reshape(info.shape)
        torch.cuda.current_stream(dev).synchronize()  # `staged` may be released once the copy has been consumed
    return out
