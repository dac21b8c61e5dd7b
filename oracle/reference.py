"""Test infrastructure: ctypes access to the checkers.

`load("ref")`   -> oracle/_ref/libgguf_ref.so, the upstream CPU REF backend compiled from the
                   upstream sources by oracle/Makefile (the parity oracle).
`load("avx2")`  -> oracle/_ref/libgguf_avx2.so, upstream's AVX2 backend (timing baseline only).
`load("port")`  -> oracle/_build/libgguf_oracle.so, this repository's plain-C restatement.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this module.
"""
from __future__ import annotations

import ctypes
from ctypes import c_bool, c_int, c_int64, c_size_t, c_void_p
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
PATHS = {
    "ref": HERE / "_ref" / "libgguf_ref.so",
    "avx2": HERE / "_ref" / "libgguf_avx2.so",
    "port": HERE / "_build" / "libgguf_oracle.so",
}


class Checker:
    """quantize_rows / dequantize_rows over one of the checker libraries, NumPy in and out."""

    def __init__(self, kind: str):
        self.kind = kind
        self.path = PATHS[kind]
        if not self.path.exists():
            raise FileNotFoundError(f"{self.path} not built: run `make -C oracle`")
        self.lib = ctypes.CDLL(str(self.path))
        prefix = "gguf_oracle_" if kind == "port" else "libgguf_"
        self._row_size = getattr(self.lib, prefix + "row_size")
        self._row_size.restype, self._row_size.argtypes = c_size_t, [c_int, c_int64]
        self._quantize = getattr(self.lib, prefix + "quantize_chunk")
        self._quantize.restype = c_size_t
        self._quantize.argtypes = [c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p]
        self._dequantize = getattr(self.lib, prefix + "dequantize_chunk")
        self._dequantize.restype = c_size_t
        self._dequantize.argtypes = [c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64]
        self._needs = getattr(self.lib, prefix + "quantize_requires_imatrix")
        self._needs.restype, self._needs.argtypes = c_bool, [c_int]

    def row_size(self, qtype: int, n_per_row: int) -> int:
        return int(self._row_size(int(qtype), int(n_per_row)))

    def requires_imatrix(self, qtype: int) -> bool:
        return bool(self._needs(int(qtype)))

    def quantize_rows(self, data: np.ndarray, qtype: int, imatrix: np.ndarray | None = None) -> np.ndarray:
        rows = np.ascontiguousarray(data, dtype=np.float32)
        n = rows.shape[-1]
        nrows = rows.size // n
        rs = self.row_size(qtype, n)
        if rs == 0:
            raise ValueError("unsupported type or row width")
        if imatrix is None and self.requires_imatrix(qtype):
            imatrix = np.sum((rows * rows).reshape(-1, n), axis=0, dtype=np.float32)
        im = None if imatrix is None else np.ascontiguousarray(imatrix, dtype=np.float32)
        out = np.empty((*rows.shape[:-1], rs), dtype=np.uint8)
        written = self._quantize(int(qtype), rows.ctypes.data, out.ctypes.data, 0, nrows, n,
                                 None if im is None else im.ctypes.data)
        if written != nrows * rs:
            raise RuntimeError(f"checker quantize wrote {written}, expected {nrows * rs}")
        return out

    def dequantize_rows(self, data: np.ndarray, qtype: int, n_per_row: int) -> np.ndarray:
        rows = np.ascontiguousarray(data, dtype=np.uint8)
        rs = rows.shape[-1]
        nrows = rows.size // rs
        out = np.empty((*rows.shape[:-1], n_per_row), dtype=np.float32)
        written = self._dequantize(int(qtype), rows.ctypes.data, out.ctypes.data, 0, nrows, n_per_row)
        if written != nrows * n_per_row * 4:
            raise RuntimeError(f"checker dequantize wrote {written}")
        return out


_cache: dict[str, Checker] = {}


def load(kind: str = "ref") -> Checker:
    if kind not in _cache:
        _cache[kind] = Checker(kind)
    return _cache[kind]


def available(kind: str) -> bool:
    return PATHS[kind].exists()
