"""Seeded input generators shared by the golden-fixture script and the tests.

`pattern_rows` reproduces the patterns of upstream bench/check_exact.py:80-118 (the inputs behind
upstream's frozen tests/golden/manifest.json).  The `*_matrix` / `conversion_tensor` functions are the
synthetic stand-ins for model weights that the benchmark workloads use: every one is a seeded NumPy
generator, so the CPU checker and the GPU see identical bits, and a row slice of the full-size matrix is
obtained by generating the full matrix and slicing it (`rows=` only changes the height for the cheap
generators whose first rows do not depend on it).  bench.py imports this module for its inputs."""
from __future__ import annotations

import numpy as np

QTYPES = {
    "Q4_0": 2, "Q4_1": 3, "Q5_0": 6, "Q5_1": 7, "Q8_0": 8, "Q2_K": 10, "Q3_K": 11, "Q4_K": 12, "Q5_K": 13,
    "Q6_K": 14, "IQ2_XXS": 16, "IQ2_XS": 17, "IQ3_XXS": 18, "IQ1_S": 19, "IQ4_NL": 20, "IQ3_S": 21, "IQ2_S": 22,
    "IQ4_XS": 23, "IQ1_M": 29, "TQ1_0": 34, "TQ2_0": 35, "MXFP4": 39, "NVFP4": 40, "Q1_0": 41,
}
BLOCK = {"Q4_0": 32, "Q4_1": 32, "Q5_0": 32, "Q5_1": 32, "Q8_0": 32, "MXFP4": 32, "IQ4_NL": 32, "NVFP4": 64, "Q1_0": 128}

PATTERNS = ("zeros", "constants", "absmax_tie_positive_first", "absmax_tie_negative_first", "outlier",
            "random_normal_seed0", "uniform", "tiny", "large", "ramp", "spikes")


def block_size(name: str) -> int:
    return BLOCK.get(name, 256)


def pattern_rows(pattern: str, rows: int, width: int, seed: int = 0) -> np.ndarray:
    rng = np.random.default_rng(seed)
    if pattern == "zeros":
        data = np.zeros((rows, width), dtype=np.float32)
    elif pattern == "constants":
        data = np.full((rows, width), 0.25, dtype=np.float32)
    elif pattern == "absmax_tie_positive_first":
        data = np.zeros((rows, width), dtype=np.float32)
        data[:, 0::4], data[:, 1::4], data[:, 2::4], data[:, 3::4] = 1.5, -1.5, 0.5, -0.5
    elif pattern == "absmax_tie_negative_first":
        data = np.zeros((rows, width), dtype=np.float32)
        data[:, 0::4], data[:, 1::4], data[:, 2::4], data[:, 3::4] = -1.5, 1.5, -0.5, 0.5
    elif pattern == "outlier":
        data = np.random.default_rng(0).normal(0.0, 0.1, size=(rows, width)).astype(np.float32)
        data[:, 0::64] = 8.0
        data[:, 1::64] = -8.0
    elif pattern == "random_normal_seed0":
        data = np.random.default_rng(0).normal(0.0, 0.75, size=(rows, width)).astype(np.float32)
    elif pattern == "uniform":
        data = rng.uniform(-2.0, 2.0, size=(rows, width)).astype(np.float32)
    elif pattern == "tiny":
        data = rng.normal(0.0, 1.0e-5, size=(rows, width)).astype(np.float32)
    elif pattern == "large":
        data = rng.normal(0.0, 16.0, size=(rows, width)).astype(np.float32)
    elif pattern == "ramp":
        data = np.linspace(-3.0, 3.0, rows * width, dtype=np.float32).reshape(rows, width)
    elif pattern == "spikes":  # constant rows with +-32 spikes (upstream test_cuda_quantize.py:122-139 style)
        data = np.full((rows, width), 0.5, dtype=np.float32)
        data[:, 7::37] = 32.0
        data[:, 11::53] = -32.0
    else:
        raise ValueError(pattern)
    return np.ascontiguousarray(data, dtype=np.float32)


def imatrix_for(width: int, seed: int = 1) -> np.ndarray:
    """Per-column importance weights, chi-square(4)/4 (the importance matrix of the lattice-quantizer workload)."""
    return (np.random.default_rng(seed).chisquare(4, width).astype(np.float32) / np.float32(4)).astype(np.float32)


def q4k_matrix(rows: int = 4096, width: int = 4096) -> np.ndarray:
    """Q4_K round-trip workload: 4096 x 4096 i.i.d. N(0, 0.02), seed 0 (first rows independent of `rows`)."""
    return (np.random.default_rng(0).standard_normal((rows, width), dtype=np.float32) * np.float32(0.02)).astype(np.float32)


def decode_sweep_matrix(rows: int = 14336, width: int = 4096) -> np.ndarray:
    """Decode-sweep workload: a 14336 x 4096 weight matrix, i.i.d. N(0, 0.02), seed 0; it is quantized by the checker
    per type and the encoded bytes are what the decoders are timed and checked on."""
    return (np.random.default_rng(0).standard_normal((rows, width), dtype=np.float32) * np.float32(0.02)).astype(np.float32)


def lattice_matrix(rows: int = 4096, width: int = 11008) -> tuple[np.ndarray, np.ndarray]:
    """Lattice-quantizer (IQ) workload: 4096 x 11008 Student-t(5) * 0.02, seed 0, with the chi-square(4)/4
    importance weights of `imatrix_for(width, 1)`."""
    x = (np.random.default_rng(0).standard_t(5, (rows, width)).astype(np.float32) * np.float32(0.02)).astype(np.float32)
    return x, imatrix_for(width, 1)


def _round_to_bf16(x: np.ndarray) -> np.ndarray:
    u = x.view(np.uint32)
    u = ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)) << np.uint32(16)
    return u.view(np.float32)


def microscaling_matrix(rows: int = 8192, width: int = 8192, seed: int = 0) -> np.ndarray:
    """MXFP4 / NVFP4 workload: Laplace(0, 0.01) rounded to bf16 and widened back to fp32; 1% of the 32-element
    blocks get one element set to +-50 sigma (sigma = 0.01 * sqrt 2)."""
    rng = np.random.default_rng(seed)
    x = _round_to_bf16(rng.laplace(0.0, 0.01, (rows, width)).astype(np.float32)).copy()
    nblocks = rows * width // 32
    chosen = rng.choice(nblocks, size=max(1, nblocks // 100), replace=False)
    pos = rng.integers(0, 32, size=chosen.size)
    sign = rng.choice(np.array([-1.0, 1.0], dtype=np.float32), size=chosen.size)
    flat = x.reshape(-1)
    flat[chosen * 32 + pos] = sign * np.float32(50 * 0.01 * np.sqrt(2.0))
    flat[:] = _round_to_bf16(flat)
    return flat.reshape(rows, width)


CONVERSION_BLOCK_ROWS = 1024


def conversion_tensor(name: str, rows: int, width: int, first_rows: int | None = None, out: np.ndarray | None = None) -> np.ndarray:
    """One tensor of the synthetic Llama-3-8B-shaped conversion set: i.i.d. N(0, 0.02) with ceil(0.1% of the columns)
    scaled by 20 as outlier channels.  The generator is seeded by the tensor's name; rows come in blocks of 1024, block b
    from `default_rng((seed, b))`, so that the blocks can be drawn by several threads (the embedding has 525 M values)
    and the first rows of a tensor do not depend on how many rows are asked for (`first_rows`).  `out` (float32,
    [rows or first_rows, width]) receives the values in place, e.g. a pinned buffer."""
    import zlib
    from concurrent.futures import ThreadPoolExecutor
    seed = zlib.crc32(name.encode())
    take = rows if first_rows is None else min(rows, first_rows)
    x = out if out is not None else np.empty((take, width), dtype=np.float32)
    assert x.shape == (take, width) and x.dtype == np.float32
    cols = np.random.default_rng((seed, 1 << 30)).choice(width, size=-(-width // 1000), replace=False)

    def fill(b: int) -> None:
        r0 = b * CONVERSION_BLOCK_ROWS
        r1 = min(take, r0 + CONVERSION_BLOCK_ROWS)
        block = x[r0:r1]
        np.random.default_rng((seed, b)).standard_normal(block.shape, dtype=np.float32, out=block)
        block *= np.float32(0.02)
        block[:, cols] *= np.float32(20.0)

    nblocks = -(-take // CONVERSION_BLOCK_ROWS)
    if nblocks <= 2:
        for b in range(nblocks):
            fill(b)
    else:
        import os
        with ThreadPoolExecutor(max_workers=min(nblocks, os.cpu_count() or 4, 16)) as pool:
            list(pool.map(fill, range(nblocks)))
    return x


# shape classes of the conversion set (name of a representative tensor, rows, width)
CONVERSION_SHAPES = (("blk.0.attn_q", 4096, 4096), ("blk.0.attn_k", 1024, 4096), ("blk.0.ffn_gate", 14336, 4096),
                     ("blk.0.ffn_down", 4096, 14336), ("token_embd", 128256, 4096))
