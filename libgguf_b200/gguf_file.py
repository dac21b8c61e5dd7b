"""GGUF v3 container: the writer the converter uses and a reader for load-time decoding.

Layout (little endian): magic "GGUF", version 3, tensor count, key/value count, the key/value pairs, the tensor
infos (name, dimensions innermost first, ggml type, offset into the data section), padding to the alignment, then
every tensor's bytes padded to the alignment.  The writer emits exactly what upstream's native converter emits
(csrc/quantize_gguf.cpp:1318-1363: string / uint32 / int64-array values, 32-byte alignment); the reader accepts every
scalar, string and array value type of the format (what upstream's src/libgguf/inspect.py:113-216 parses).
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field

import numpy as np

GGUF_MAGIC = 0x46554747
GGUF_VERSION = 3
DEFAULT_ALIGNMENT = 32

# value type codes of the format
T_UINT8, T_INT8, T_UINT16, T_INT16, T_UINT32, T_INT32, T_FLOAT32, T_BOOL, T_STRING, T_ARRAY, T_UINT64, T_INT64, T_FLOAT64 = range(13)
_SCALAR_FORMATS = {T_UINT8: "<B", T_INT8: "<b", T_UINT16: "<H", T_INT16: "<h", T_UINT32: "<I", T_INT32: "<i", T_FLOAT32: "<f",
                   T_BOOL: "<?", T_UINT64: "<Q", T_INT64: "<q", T_FLOAT64: "<d"}


def pad_to(n: int, alignment: int = DEFAULT_ALIGNMENT) -> int:
    return (n + alignment - 1) // alignment * alignment


def _string(value: str) -> bytes:
    raw = value.encode("utf-8")
    return struct.pack("<Q", len(raw)) + raw


@dataclass
class TensorInfo:
    name: str
    shape: tuple[int, ...]      # outermost first (row-major), as in the source checkpoint
    qtype: int
    nbytes: int
    offset: int = 0             # relative to the start of the data section


def encode_kv(key: str, value_type: int, value) -> bytes:
    out = _string(key) + struct.pack("<I", value_type)
    if value_type == T_STRING:
        return out + _string(value)
    if value_type == T_ARRAY:
        element_type, items = value
        out += struct.pack("<IQ", element_type, len(items))
        if element_type == T_STRING:
            return out + b"".join(_string(v) for v in items)
        return out + b"".join(struct.pack(_SCALAR_FORMATS[element_type], v) for v in items)
    return out + struct.pack(_SCALAR_FORMATS[value_type], value)


def header_bytes(kv: list[tuple[str, int, object]], infos: list[TensorInfo], alignment: int = DEFAULT_ALIGNMENT) -> bytes:
    """Everything before the data section, without the trailing padding.  Fills in the tensor offsets."""
    out = [struct.pack("<IIQQ", GGUF_MAGIC, GGUF_VERSION, len(infos), len(kv))]
    out += [encode_kv(k, t, v) for k, t, v in kv]
    offset = 0
    for info in infos:
        info.offset = offset
        out.append(_string(info.name) + struct.pack("<I", len(info.shape)))
        out.append(b"".join(struct.pack("<Q", d) for d in reversed(info.shape)))
        out.append(struct.pack("<IQ", info.qtype, offset))
        offset += pad_to(info.nbytes, alignment)
    return b"".join(out)


@dataclass
class GGUFFile:
    path: str
    version: int
    metadata: dict = field(default_factory=dict)
    tensors: dict = field(default_factory=dict)   # name -> TensorInfo
    data_start: int = 0
    alignment: int = DEFAULT_ALIGNMENT

    def tensor_bytes(self, name: str) -> np.ndarray:
        """The tensor's stored bytes as a read-only memory map (no copy)."""
        info = self.tensors[name]
        return np.memmap(self.path, dtype=np.uint8, mode="r", offset=self.data_start + info.offset, shape=(info.nbytes,))


class _Cursor:
    def __init__(self, data: memoryview):
        self.data, self.pos = data, 0

    def take(self, fmt: str):
        size = struct.calcsize(fmt)
        if self.pos + size > len(self.data):
            raise ValueError("truncated GGUF header")
        (value,) = struct.unpack_from(fmt, self.data, self.pos)
        self.pos += size
        return value

    def string(self) -> str:
        n = self.take("<Q")
        if self.pos + n > len(self.data):
            raise ValueError("truncated GGUF string")
        raw = bytes(self.data[self.pos:self.pos + n])
        self.pos += n
        return raw.decode("utf-8", errors="replace")

    def value(self, value_type: int):
        if value_type == T_STRING:
            return self.string()
        if value_type == T_ARRAY:
            element_type, count = self.take("<I"), self.take("<Q")
            return [self.value(element_type) for _ in range(count)]
        if value_type not in _SCALAR_FORMATS:
            raise ValueError(f"unknown GGUF value type {value_type}")
        return self.take(_SCALAR_FORMATS[value_type])


def read_gguf(path: str, row_size=None) -> GGUFFile:
    """Parses header, metadata and tensor infos.  `row_size(qtype, n_per_row)` (e.g. libgguf_b200.row_size) gives
    each tensor's byte size; without it sizes are taken from the distance to the next tensor."""
    with open(path, "rb") as f:
        head = f.read(24)
        if len(head) < 24:
            raise ValueError("not a GGUF file")
        magic, version, n_tensors, n_kv = struct.unpack("<IIQQ", head)
        if magic != GGUF_MAGIC:
            raise ValueError("not a GGUF file")
        if version not in (2, 3):
            raise ValueError(f"unsupported GGUF version {version}")
    data = np.memmap(path, dtype=np.uint8, mode="r")
    cur = _Cursor(memoryview(data))
    cur.pos = 24
    out = GGUFFile(path=path, version=version)
    for _ in range(n_kv):
        key = cur.string()
        out.metadata[key] = cur.value(cur.take("<I"))
    out.alignment = int(out.metadata.get("general.alignment", DEFAULT_ALIGNMENT))
    infos = []
    for _ in range(n_tensors):
        name = cur.string()
        n_dims = cur.take("<I")
        dims = [cur.take("<Q") for _ in range(n_dims)]
        qtype, offset = cur.take("<I"), cur.take("<Q")
        infos.append(TensorInfo(name=name, shape=tuple(reversed(dims)), qtype=qtype, nbytes=0, offset=offset))
    out.data_start = pad_to(cur.pos, out.alignment)
    data_size = len(data) - out.data_start
    by_offset = sorted(infos, key=lambda t: t.offset)
    for i, info in enumerate(by_offset):
        limit = (by_offset[i + 1].offset if i + 1 < len(by_offset) else data_size) - info.offset
        if row_size is not None:
            n_per_row = info.shape[-1] if info.shape else 1
            rows = int(np.prod(info.shape[:-1], dtype=np.int64)) if len(info.shape) > 1 else 1
            info.nbytes = rows * row_size(info.qtype, n_per_row)
            if info.nbytes == 0 or info.nbytes > limit:
                raise ValueError(f"tensor {info.name} does not fit its slot in the file")
        else:
            info.nbytes = limit
        out.tensors[info.name] = info
    return out
