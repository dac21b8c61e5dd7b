"""Seeded input generators shared by the golden-fixture script and the tests.

`pattern_rows` reproduces the patterns of upstream bench/check_exact.py:80-118 (the inputs behind
upstream's frozen tests/golden/manifest.json); the `config_*` functions are the synthetic
stand-ins for the BASELINE configurations."""
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
    """Per-column importance weights, chi-square(4)/4 as in BASELINE config 4."""
    return (np.random.default_rng(seed).chisquare(4, width).astype(np.float32) / np.float32(4)).astype(np.float32)


def config1(rows: int = 4096, width: int = 4096) -> np.ndarray:
    return (np.random.default_rng(0).standard_normal((rows, width), dtype=np.float32) * np.float32(0.02)).astype(np.float32)


def config4(rows: int = 4096, width: int = 11008) -> tuple[np.ndarray, np.ndarray]:
    x = (np.random.default_rng(0).standard_t(5, (rows, width)).astype(np.float32) * np.float32(0.02)).astype(np.float32)
    return x, imatrix_for(width, 1)


def config5(rows: int = 8192, width: int = 8192, seed: int = 0) -> np.ndarray:
    """Laplace(0, 0.01) rounded to bf16 and widened; 1% of 32-element blocks get one +-50 sigma outlier."""
    rng = np.random.default_rng(seed)
    x = rng.laplace(0.0, 0.01, (rows, width)).astype(np.float32)
    u = x.view(np.uint32)
    u = ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)) << np.uint32(16)
    x = u.view(np.float32).copy()
    nblocks = rows * width // 32
    chosen = rng.choice(nblocks, size=max(1, nblocks // 100), replace=False)
    pos = rng.integers(0, 32, size=chosen.size)
    sign = rng.choice(np.array([-1.0, 1.0], dtype=np.float32), size=chosen.size)
    flat = x.reshape(-1)
    flat[chosen * 32 + pos] = sign * np.float32(50 * 0.01 * np.sqrt(2.0))
    u = flat.view(np.uint32)
    flat[:] = (((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)) << np.uint32(16)).view(np.float32)
    return flat.reshape(rows, width)
