"""Type tables of the C ABI against the Python tables and against the upstream library
(upstream tests/test_metadata_contracts.py:40-79)."""
import pytest

import libgguf_b200 as g
from libgguf_b200 import GGMLQuantizationType as Q, GGML_QUANT_SIZES

ROW_TYPES = [q for q in Q if q not in (Q.Q8_1, Q.Q8_K, Q.I8, Q.I16, Q.I32, Q.I64, Q.F64)]


@pytest.mark.parametrize("q", list(Q))
def test_type_size_matches_table(q):
    assert g.type_size(q) == GGML_QUANT_SIZES[q][1]


@pytest.mark.parametrize("q", ROW_TYPES)
def test_row_size(q):
    block, size = GGML_QUANT_SIZES[q]
    assert g.row_size(q, block * 3) == 3 * size
    assert g.row_size(q, 0) == 0
    assert g.row_size(q, -block) == 0
    if block > 1:
        assert g.row_size(q, block + 1) == 0


def test_unknown_types():
    for code in (4, 5, 31, 32, 33, 36, 37, 38, 42, 99, -1):
        assert g.type_size(code) == 0
        assert g.type_name(code) == "unknown"
        assert g.row_size(code, 256) == 0
    for q in (Q.Q8_1, Q.Q8_K, Q.I8, Q.F64):
        assert g.row_size(q, 256) == 0


def test_imatrix_required_set():
    assert {q for q in Q if g.quantize_requires_imatrix(q)} == {Q.IQ2_XXS, Q.IQ2_XS, Q.IQ1_S}


def test_names():
    assert g.type_name(Q.Q4_K) == "q4_K"
    assert g.type_name(Q.IQ2_XXS) == "iq2_xxs"
    assert g.type_name(Q.BF16) == "bf16"


def test_tables_match_upstream_library(ref):
    import ctypes
    lib = ref.lib
    lib.libgguf_type_size.restype = ctypes.c_size_t
    lib.libgguf_type_name.restype = ctypes.c_char_p
    for code in range(-1, 45):
        assert g.type_size(code) == lib.libgguf_type_size(code), code
        assert g.type_name(code) == lib.libgguf_type_name(code).decode(), code
        for n in (1, 31, 32, 64, 128, 256, 4096, 4097):
            assert g.row_size(code, n) == ref.row_size(code, n), (code, n)
        assert g.quantize_requires_imatrix(code) == ref.requires_imatrix(code)
