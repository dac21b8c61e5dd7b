"""Multi-GPU streaming conversion: the converter's tensor loop over the C-ABI pipeline.

`ConversionPipeline` wraps libgguf_cuda_pipeline_* (csrc/pipeline.cu): a batch of host tensors is cut into
row-range shards and streamed through every listed GPU with no GPU-to-GPU traffic.  `llama3_8b_plan` is the
synthetic stand-in for the Llama-3-8B weight set of the conversion benchmark (shapes and the Q4_K_M-style
type mix only; the values are generated, no checkpoint is involved).

upstream counterpart: csrc/quantize_gguf.cpp:1990-2223 (write_tensor_payload) driven by the plan of
:1235-1316; upstream runs it on GPU 0 with two pinned slots."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import numpy as np

from . import GGMLQuantizationType, row_size
from ._native import ShardDesc, TensorDesc, lib


# numpy dtype of a source array -> source dtype code of the C ABI (bfloat16 travels as uint16 bit patterns)
SOURCE_DTYPES = {np.dtype(np.float32): 0, np.dtype(np.float16): 1, np.dtype(np.uint16): 2}


@dataclass
class PlannedTensor:
    name: str
    rows: int
    cols: int
    qtype: int


def llama3_8b_plan(n_layers: int = 32) -> list[PlannedTensor]:
    """Tensor list of a Llama-3-8B-shaped model with the Q4_K_M mix: Q6_K for `output` and for `attn_v` and
    `ffn_down` of every second layer, Q4_K elsewhere."""
    q4, q6 = int(GGMLQuantizationType.Q4_K), int(GGMLQuantizationType.Q6_K)
    plan = [PlannedTensor("token_embd", 128256, 4096, q4)]
    for layer in range(n_layers):
        more_bits = layer % 2 == 0
        plan += [
            PlannedTensor(f"blk.{layer}.attn_q", 4096, 4096, q4),
            PlannedTensor(f"blk.{layer}.attn_k", 1024, 4096, q4),
            PlannedTensor(f"blk.{layer}.attn_v", 1024, 4096, q6 if more_bits else q4),
            PlannedTensor(f"blk.{layer}.attn_output", 4096, 4096, q4),
            PlannedTensor(f"blk.{layer}.ffn_gate", 14336, 4096, q4),
            PlannedTensor(f"blk.{layer}.ffn_up", 14336, 4096, q4),
            PlannedTensor(f"blk.{layer}.ffn_down", 4096, 14336, q6 if more_bits else q4),
        ]
    plan.append(PlannedTensor("output", 128256, 4096, q6))
    return plan


class ConversionPipeline:
    def __init__(self, devices: list[int], slots: int = 3, chunk_bytes: int = 128 << 20):
        self.devices = list(devices)
        arr = (ctypes.c_int * len(self.devices))(*self.devices)
        self._handle = ctypes.c_void_p()
        status = lib.libgguf_cuda_pipeline_create(arr, len(self.devices), slots, chunk_bytes, ctypes.byref(self._handle))
        if status != 0:
            raise RuntimeError(f"libgguf_cuda_pipeline_create failed with status {status}")

    def close(self) -> None:
        if self._handle:
            lib.libgguf_cuda_pipeline_destroy(self._handle)
            self._handle = ctypes.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    @staticmethod
    def _descs(tensors):
        keep = []
        descs = (TensorDesc * len(tensors))()
        dtypes = (ctypes.c_int32 * len(tensors))()
        for i, (d, (qtype, src, imatrix, dst)) in enumerate(zip(descs, tensors)):
            if src.dtype not in SOURCE_DTYPES or src.ndim != 2 or not src.flags.c_contiguous:
                raise ValueError("src must be a C-contiguous 2-D array of float32, float16, or uint16 holding bfloat16 bits")
            dtypes[i] = SOURCE_DTYPES[src.dtype]
            if dst.dtype != np.uint8 or not dst.flags.c_contiguous or not dst.flags.writeable:
                raise ValueError("dst must be a writable C-contiguous uint8 array")
            rs = row_size(qtype, src.shape[1])
            if rs == 0 or dst.size != src.shape[0] * rs:
                raise ValueError("dst size does not match rows * row_size for this type")
            im = None
            if imatrix is not None:
                im = np.ascontiguousarray(imatrix, dtype=np.float32)
                if im.shape != (src.shape[1],):
                    raise ValueError("imatrix length must match n_per_row")
                keep.append(im)
            d.qtype, d.src, d.imatrix, d.dst = int(qtype), src.ctypes.data, (im.ctypes.data if im is not None else None), dst.ctypes.data
            d.rows, d.n_per_row = src.shape
        return descs, dtypes, keep

    def quantize(self, tensors) -> None:
        """tensors: list of (qtype, src [rows, n], imatrix or None, dst uint8 [rows * row_size]).  `src` is float32, or
        float16 / uint16-as-bfloat16, in which case the 16-bit values are uploaded as they are and widened on the GPU."""
        descs, dtypes, keep = self._descs(tensors)
        status = lib.libgguf_cuda_pipeline_quantize_typed(self._handle, descs, dtypes, len(tensors))
        if status != 0:
            raise RuntimeError(f"pipeline failed (status {status}): {lib.libgguf_cuda_pipeline_last_error(self._handle).decode()}")

    def inject_failure(self, device_slot: int, after_shards: int) -> None:
        if lib.libgguf_cuda_pipeline_inject_failure(self._handle, device_slot, after_shards) != 0:
            raise ValueError("bad device slot")

    def stats(self) -> dict:
        n = len(self.devices)
        shards = (ctypes.c_int64 * n)()
        secs = (ctypes.c_double * n)()
        requeued = ctypes.c_int64()
        lib.libgguf_cuda_pipeline_stats(self._handle, shards, secs, ctypes.byref(requeued))
        return {"shards_per_device": list(shards), "seconds_per_device": list(secs), "requeued": requeued.value}


def whole_tensor_imatrix(src: np.ndarray) -> np.ndarray:
    """Column sums of squares over ALL rows of a 2-D source (float32, float16, or uint16 holding bfloat16 bits), added
    in row order on the GPU: the importance weights upstream derives for a type that requires them when the caller
    has none (upstream csrc/_libgguf_module.cpp:1210-1242, src/libgguf/__init__.py:186-189).  Whoever cuts a tensor into
    row pieces computes this once and hands it to every piece."""
    if src.dtype not in SOURCE_DTYPES or src.ndim != 2 or not src.flags.c_contiguous:
        raise ValueError("src must be a C-contiguous 2-D array of float32, float16, or uint16 holding bfloat16 bits")
    out = np.zeros(src.shape[1], dtype=np.float32)
    status = lib.libgguf_cuda_auto_imatrix_typed(src.ctypes.data, SOURCE_DTYPES[src.dtype], src.shape[0], src.shape[1], out.ctypes.data)
    if status != 0:
        raise RuntimeError(f"libgguf_cuda_auto_imatrix_typed failed with status {status}")
    return out


def plan_shards(tensors: list[tuple[int, int, int]], chunk_bytes: int = 128 << 20, source_dtypes=None) -> list[tuple[int, int, int]]:
    """Shard list for tensors given as (qtype, rows, n_per_row); needs no GPU.  Returns (tensor, row0, rows).
    source_dtypes: optional list of 0 (float32), 1 (float16), 2 (bfloat16); a shard holds at most chunk_bytes of source."""
    descs = (TensorDesc * len(tensors))()
    for d, (qtype, rows, n) in zip(descs, tensors):
        d.qtype, d.rows, d.n_per_row = int(qtype), rows, n
    dtypes = (ctypes.c_int32 * len(tensors))(*source_dtypes) if source_dtypes is not None else None
    count = lib.libgguf_cuda_pipeline_plan_typed(descs, dtypes, len(tensors), chunk_bytes, None, 0)
    if count < 0:
        raise ValueError("bad tensor descriptor")
    out = (ShardDesc * count)()
    lib.libgguf_cuda_pipeline_plan_typed(descs, dtypes, len(tensors), chunk_bytes, out, count)
    return [(s.tensor, s.row0, s.rows) for s in out]


def assign_shards(shards: list[tuple[int, int, int]], widths: list[int], world: int,
                  rates: list[float] | None = None) -> list[list[tuple[int, int, int]]]:
    """Split a shard list over `world` processes (one per GPU) without any exchange of data: shards are taken in the
    given (largest-first) order and each goes to the process that would finish it earliest, lowest rank on ties.
    Every process computes the same answer from the same plan, so no rank needs to talk to another.
    `widths[t]` is n_per_row of tensor t.  `rates` (optional, one positive number per process, e.g. the host-to-device
    rate each process measured on its own link at start-up and all processes exchanged once) weights the shares: a
    process behind a link of half the rate gets half the elements.  Without it every process counts the same."""
    if world < 1:
        raise ValueError("world must be positive")
    if rates is None:
        rates = [1.0] * world
    if len(rates) != world or any(not (r > 0) for r in rates):
        raise ValueError("rates must hold one positive number per process")
    load = [0.0] * world
    out: list[list[tuple[int, int, int]]] = [[] for _ in range(world)]
    for shard in shards:
        tensor, _, rows = shard
        work = rows * widths[tensor]
        r = min(range(world), key=lambda i: ((load[i] + work) / rates[i], i))
        out[r].append(shard)
        load[r] += work
    return out


def rank_batch(tensors, world: int, rank: int, chunk_bytes: int = 128 << 20, rates: list[float] | None = None):
    """The slice of a conversion batch that process `rank` of `world` runs on its own GPU.
    tensors: list of (qtype, src float32 [rows, n], imatrix or None, dst uint8 [rows * row_size]); the result has the
    same form, with `src` and `dst` replaced by row-range views, and can be given to ConversionPipeline.quantize."""
    shards = plan_shards([(q, s.shape[0], s.shape[1]) for q, s, _, _ in tensors], chunk_bytes,
                         [SOURCE_DTYPES[s.dtype] for _, s, _, _ in tensors])
    mine = assign_shards(shards, [s.shape[1] for _, s, _, _ in tensors], world, rates)[rank]
    batch = []
    derived: dict[int, np.ndarray] = {}
    for tensor, row0, rows in mine:
        qtype, src, imatrix, dst = tensors[tensor]
        if imatrix is None and lib.libgguf_quantize_requires_imatrix(int(qtype)) and rows != src.shape[0]:
            # a row range of a tensor whose type needs importance weights: they come from the whole tensor, which
            # every rank can compute for itself (no exchange), never from the rank's own slice
            if tensor not in derived:
                derived[tensor] = whole_tensor_imatrix(src)
            imatrix = derived[tensor]
        rs = row_size(qtype, src.shape[1])
        batch.append((qtype, src[row0:row0 + rows], imatrix, dst[row0 * rs:(row0 + rows) * rs]))
    return batch


def max_over_ranks(value: float, device=None) -> float:
    """The slowest rank's `value` (a duration) when torch.distributed is initialised, else `value`."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device if device is not None else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
