"""Pins the checkers: the compiled upstream REF backend and this repository's C restatement
must reproduce upstream's 70 frozen hashes and the golden fixtures generated from upstream."""
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest

import inputs

GOLDEN = Path(__file__).parent / "golden"
UPSTREAM = json.loads((GOLDEN / "upstream_manifest.json").read_text())["entries"]
FIXTURES = json.loads((GOLDEN / "golden.json").read_text())["entries"]

PORTED = None  # filled from the oracle library


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def upstream_case(e):
    rows, width = (int(v) for v in e["shape"].split("x"))
    return inputs.pattern_rows(e["pattern"], rows, width), inputs.QTYPES[e["qtype"]]


def fixture_case(e):
    qtype = inputs.QTYPES[e["qtype"]]
    x = inputs.pattern_rows(e["pattern"], e["rows"], e["width"], seed=qtype * 1009 + sum(e["pattern"].encode()))
    im = inputs.imatrix_for(e["width"], seed=qtype) if e["weighted"] else None
    return x, qtype, im


def test_reference_build_reproduces_upstream_manifest(ref):
    assert len(UPSTREAM) == 70
    for e in UPSTREAM:
        x, qtype = upstream_case(e)
        enc = ref.quantize_rows(x, qtype)
        assert enc.nbytes == e["encoded_nbytes"]
        assert sha(enc) == e["encoded_sha256"], e


def test_reference_build_reproduces_fixtures(ref):
    for e in FIXTURES:
        x, qtype, im = fixture_case(e)
        enc = ref.quantize_rows(x, qtype, im)
        assert sha(enc) == e["encoded_sha256"], e
        assert sha(ref.dequantize_rows(enc, qtype, e["width"])) == e["decoded_sha256"], e


def _port_supports(port, qtype):
    return port.lib.gguf_oracle_quantize_supported(int(qtype)) != 0


def test_port_reproduces_upstream_manifest(port):
    checked = 0
    for e in UPSTREAM:
        x, qtype = upstream_case(e)
        if not _port_supports(port, qtype):
            continue
        assert sha(port.quantize_rows(x, qtype)) == e["encoded_sha256"], e
        checked += 1
    assert checked >= 50


def test_port_reproduces_fixtures(port):
    checked = 0
    for e in FIXTURES:
        x, qtype, im = fixture_case(e)
        if _port_supports(port, qtype):
            enc = port.quantize_rows(x, qtype, im)
            assert sha(enc) == e["encoded_sha256"], e
            checked += 1
    assert checked > 0


def test_port_decoders_reproduce_fixtures(port, ref):
    """Every decoder of the restatement, on reference-encoded bytes."""
    for e in FIXTURES:
        if e["weighted"]:
            continue
        x, qtype, im = fixture_case(e)
        enc = ref.quantize_rows(x, qtype, im)
        assert sha(port.dequantize_rows(enc, qtype, e["width"])) == e["decoded_sha256"], e


@pytest.mark.parametrize("name", ["Q8_0", "Q4_K", "Q6_K", "Q2_K", "MXFP4", "NVFP4"])
def test_port_matches_reference_on_random_rows(port, ref, name):
    qtype = inputs.QTYPES[name]
    if not _port_supports(port, qtype):
        pytest.skip("not restated yet")
    x = (np.random.default_rng(7).standard_normal((32, 2048)) * 0.02).astype(np.float32)
    np.testing.assert_array_equal(port.quantize_rows(x, qtype), ref.quantize_rows(x, qtype))
