"""Parity of the CUDA path with the checkers, through the C ABI.

Encoded bytes must be identical; fp32 decodes must have identical bit patterns; fp16/bf16
decodes must equal the round-to-nearest-even conversion of the fp32 decode (bit patterns)."""
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest

import inputs

pytestmark = pytest.mark.gpu

GOLDEN = Path(__file__).parent / "golden"
UPSTREAM = json.loads((GOLDEN / "upstream_manifest.json").read_text())["entries"]
FIXTURES = json.loads((GOLDEN / "golden.json").read_text())["entries"]
ALL = sorted(inputs.QTYPES)


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.fixture(scope="module")
def checker():
    from oracle import reference
    if reference.available("ref"):
        return reference.load("ref")
    import subprocess
    if not reference.available("port"):
        subprocess.run(["make", "-C", str(Path(__file__).parents[1] / "oracle"), "oracle"], check=True, capture_output=True)
    return reference.load("port")


def supported_by(checker, qtype):
    if checker.kind == "port":
        return checker.lib.gguf_oracle_quantize_supported(int(qtype)) != 0
    return True


def test_upstream_frozen_vectors(gguf):
    """The 70 SHA-256 vectors upstream freezes for its CPU backend (tests/golden/manifest.json)."""
    for e in UPSTREAM:
        rows, width = (int(v) for v in e["shape"].split("x"))
        x = inputs.pattern_rows(e["pattern"], rows, width)
        enc = gguf.quantize_rows(x, inputs.QTYPES[e["qtype"]])
        assert enc.nbytes == e["encoded_nbytes"]
        assert sha(enc) == e["encoded_sha256"], e
        dec = gguf.dequantize_rows(enc, inputs.QTYPES[e["qtype"]], width)
        assert np.all(np.isfinite(dec))


@pytest.mark.parametrize("name", ALL)
def test_golden_fixtures(gguf, name):
    """Every type x 11 patterns x {no imatrix, imatrix}: encoded bytes and fp32 decode."""
    n = 0
    for e in FIXTURES:
        if e["qtype"] != name:
            continue
        qtype = inputs.QTYPES[name]
        x = inputs.pattern_rows(e["pattern"], e["rows"], e["width"], seed=qtype * 1009 + sum(e["pattern"].encode()))
        im = inputs.imatrix_for(e["width"], seed=qtype) if e["weighted"] else None
        enc = gguf.quantize_rows(x, qtype, im)
        assert sha(enc) == e["encoded_sha256"], e
        assert sha(gguf.dequantize_rows(enc, qtype, e["width"])) == e["decoded_sha256"], e
        n += 1
    assert n == 2 * len(inputs.PATTERNS)


@pytest.mark.parametrize("name", ALL)
def test_random_rows_match_checker(gguf, checker, name):
    """512 x 4096 standard normal rows, seed 0 (upstream test_cuda_quantize.py:279-311 shape)."""
    qtype = inputs.QTYPES[name]
    if not supported_by(checker, qtype):
        pytest.skip("checker has no quantizer for this type")
    slow = name.startswith("IQ1") or name.startswith("IQ2") or name.startswith("IQ3")
    rows = 64 if slow else 512
    x = np.random.default_rng(0).standard_normal((rows, 4096), dtype=np.float32)
    want = checker.quantize_rows(x, qtype)
    got = gguf.quantize_rows(x, qtype)
    bad_rows = np.flatnonzero((want != got).any(axis=-1))
    assert bad_rows.size == 0, f"{bad_rows.size} rows differ, first {bad_rows[:5]}"
    np.testing.assert_array_equal(gguf.dequantize_rows(want, qtype, 4096).view(np.uint32),
                                  checker.dequantize_rows(want, qtype, 4096).view(np.uint32))


@pytest.mark.parametrize("name", ["Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K", "IQ4_NL", "IQ4_XS",
                                  "IQ2_XXS", "IQ2_XS", "IQ2_S", "IQ3_XXS", "IQ3_S", "IQ1_S", "IQ1_M"])
def test_importance_weighted_rows_match_checker(gguf, checker, name):
    qtype = inputs.QTYPES[name]
    if not supported_by(checker, qtype):
        pytest.skip("checker has no quantizer for this type")
    x, im = inputs.lattice_matrix(32, 2048)
    np.testing.assert_array_equal(gguf.quantize_rows(x, qtype, im), checker.quantize_rows(x, qtype, im))


@pytest.mark.parametrize("name", ["IQ2_XXS", "IQ2_XS", "IQ2_S", "IQ3_XXS", "IQ3_S", "IQ1_S", "IQ1_M"])
def test_lattice_workload_slice_at_full_width(gguf, checker, name):
    """The lattice-quantizer benchmark workload at its own width: a 256-row slice of the 4096 x 11008 Student-t matrix with the
    chi-square importance weights, plus rows whose blocks are partly zero (lanes that queue no scans next to lanes
    that queue long ones) and one row of large outliers."""
    qtype = inputs.QTYPES[name]
    if not supported_by(checker, qtype):
        pytest.skip("checker has no quantizer for this type")
    x, im = inputs.lattice_matrix(256, 11008)
    x = x.copy()
    x[3, 256:1024] = 0.0
    x[4, ::2] = 0.0
    x[5, 32:64] = 0.0
    x[6, ::97] *= np.float32(400.0)
    want = checker.quantize_rows(x, qtype, im)
    got = gguf.quantize_rows(x, qtype, im)
    bad_rows = np.flatnonzero((want != got).any(axis=-1))
    assert bad_rows.size == 0, f"{bad_rows.size} rows differ, first {bad_rows[:5]}"


@pytest.mark.parametrize("name", ALL)
def test_ragged_sizes_and_chunk_offsets(gguf, checker, name):
    """1 block, 1 row, row counts that do not fill a CTA, and start offsets into a larger matrix."""
    from libgguf_b200._native import lib
    qtype = inputs.QTYPES[name]
    if not supported_by(checker, qtype):
        pytest.skip("checker has no quantizer for this type")
    block = inputs.block_size(name)
    rng = np.random.default_rng(5)
    for rows, width in ((1, block), (3, block * 3), (7, block * 5), (33, block)):
        x = rng.standard_normal((rows, width), dtype=np.float32)
        np.testing.assert_array_equal(gguf.quantize_rows(x, qtype), checker.quantize_rows(x, qtype))
    # chunked call: rows 5..11 of a 16-row matrix land at their own offset, the rest untouched
    width = block * 4
    x = rng.standard_normal((16, width), dtype=np.float32)
    want = checker.quantize_rows(x, qtype)
    im = None
    if checker.requires_imatrix(qtype):
        im = np.sum(x * x, axis=0, dtype=np.float32)
    out = np.full_like(want, 0xAB)
    rs = want.shape[-1]
    n = lib.libgguf_quantize_chunk(qtype, x.ctypes.data, out.ctypes.data, 5 * width, 6, width,
                                   None if im is None else im.ctypes.data)
    assert n == 6 * rs
    np.testing.assert_array_equal(out[5:11], want[5:11])
    assert (out[:5] == 0xAB).all() and (out[11:] == 0xAB).all()
    dec = np.full((16, width), np.float32(-7), np.float32)
    n = lib.libgguf_dequantize_chunk(qtype, want.ctypes.data, dec.ctypes.data, 5 * width, 6, width)
    assert n == 6 * width * 4
    np.testing.assert_array_equal(dec[5:11].view(np.uint32), checker.dequantize_rows(want[5:11], qtype, width).view(np.uint32))
    assert (dec[:5] == -7).all() and (dec[11:] == -7).all()


def test_q4k_roundtrip_workload_properties(gguf, checker):
    """The Q4_K round-trip workload at full size (4096 x 4096, N(0, 0.02), seed 0): bytes against the checker
    on a 256-row slice; on the whole matrix, chunk independence (any row range encodes to the same
    bytes as in the full call) and idempotence of decode -> encode -> decode."""
    x = inputs.q4k_matrix()
    enc = gguf.quantize_rows(x, 12)
    np.testing.assert_array_equal(enc[1000:1256], checker.quantize_rows(x[1000:1256], 12))
    np.testing.assert_array_equal(enc[17:83], gguf.quantize_rows(x[17:83], 12))
    dec = gguf.dequantize_rows(enc, 12, 4096)
    np.testing.assert_array_equal(dec[1000:1256].view(np.uint32),
                                  checker.dequantize_rows(enc[1000:1256], 12, 4096).view(np.uint32))
    err = np.abs(dec - x).max()
    assert err < 0.02 * 0.6
    dec2 = gguf.dequantize_rows(gguf.quantize_rows(dec, 12), 12, 4096)
    assert np.abs(dec2 - dec).max() <= err


def test_storage_types(gguf, checker):
    x = np.random.default_rng(3).standard_normal((5, 96), dtype=np.float32)
    x[0, :4] = [np.inf, -np.inf, np.nan, 1e-8]
    assert np.array_equal(gguf.quantize_rows(x, 0).view(np.uint32), x.view(np.uint32))
    h = gguf.quantize_rows(x, 1)
    assert h.dtype == np.float16 and h.shape == x.shape
    if checker.kind == "ref":
        np.testing.assert_array_equal(h.view(np.uint16).reshape(5, -1), checker.quantize_rows(x, 1).view(np.uint16))
        np.testing.assert_array_equal(gguf.quantize_rows(x, 30), checker.quantize_rows(x, 30))
    else:
        finite = np.isfinite(x)
        np.testing.assert_array_equal(h[finite], x.astype(np.float16)[finite])


def test_zero_rows_and_empty(gguf):
    out = gguf.quantize_rows(np.zeros((0, 256), np.float32), 12)
    assert out.shape == (0, 144)
    assert gguf.dequantize_rows(np.zeros((0, 144), np.uint8), 12).shape == (0, 256)


def test_fp4_threshold_search_equals_the_scan_for_every_float():
    """All 2^32 inputs at each scale: zero, the smallest and a mid E8M0 half-scale, UE4M3 scales with mantissa
    bits (smallest subnormal, 1.875 * 2^-1, the largest), and a huge E8M0 scale."""
    import ctypes
    from libgguf_b200._native import lib
    scales = [0.0, 2.0 ** -128, 2.0 ** -20, 0.5, 2.0 ** -10, 1.875 * 0.25, 224.0, 0.0068359375, 2.0 ** 100]
    for e in scales:
        bad = ctypes.c_uint64(123)
        assert lib.libgguf_cuda_selftest_fp4(e, ctypes.byref(bad)) == 0
        assert bad.value == 0, (e, bad.value)


def test_hardware_fp4_conversion_paths_equal_the_scan_for_every_float():
    """The MXFP4 form (power-of-two scales, smallest to largest it is used for) and the NVFP4 form (UE4M3 scales with
    and without mantissa bits) over all 2^32 inputs."""
    import ctypes
    from libgguf_b200._native import lib
    for e in (2.0 ** -128, 2.0 ** -127, 2.0 ** -126, 2.0 ** -20, 0.5, 1.0, 2.0 ** 100, 2.0 ** 124):
        bad = ctypes.c_uint64(123)
        assert lib.libgguf_cuda_selftest_fp4_mode(e, 1, ctypes.byref(bad), None) == 0
        assert bad.value == 0, (e, bad.value)
    assert lib.libgguf_cuda_selftest_fp4_mode(3.0, 1, ctypes.byref(bad), None) != 0  # not a power of two
    for e in (2.0 ** -10, 7 * 2.0 ** -10, 2.0 ** -7, 1.875 * 0.25, 0.5, 1.125, 224.0, 0.0068359375):
        bad, fell = ctypes.c_uint64(123), ctypes.c_uint64(123)
        assert lib.libgguf_cuda_selftest_fp4_mode(e, 2, ctypes.byref(bad), ctypes.byref(fell)) == 0
        assert bad.value == 0, (e, bad.value)
        assert fell.value < 2000, (e, fell.value)  # a few bit patterns around each of the 14 signed ties


def _edge_rows(width=256):
    """Blocks that leave the fast encoders: signed zeros, equal-magnitude extrema, denormal scales whose
    reciprocal overflows, exact FP4 ties, infinities, and (last rows) NaN."""
    rng = np.random.default_rng(11)
    rows = []
    z = np.zeros(width, np.float32); z[1::2] = -0.0; rows.append(z)
    z = np.zeros(width, np.float32); z[0::3] = -0.0; z[5::7] = 1.25; rows.append(z)            # min is a zero
    z = np.zeros(width, np.float32); z[0::3] = -0.0; z[5::7] = -1.25; z[2] = 0.0; rows.append(z)  # max is a zero
    z = rng.standard_normal(width).astype(np.float32); z[3::32] = 4.0; z[9::32] = -4.0; rows.append(z)   # +a before -a
    z = rng.standard_normal(width).astype(np.float32); z[3::32] = -4.0; z[9::32] = 4.0; rows.append(z)   # -a before +a
    rows.append((rng.standard_normal(width) * 1e-42).astype(np.float32))
    rows.append((rng.standard_normal(width) * 1e-38).astype(np.float32))
    rows.append((rng.standard_normal(width) * 1e37).astype(np.float32))
    ties = np.array([0.5, 1.5, 2.5, 3.5, 5.0, 7.0, 10.0, -0.5, -1.5, -2.5, -3.5, -5.0, -7.0, -10.0, 12.0, -12.0], np.float32)
    for scale in (1.0, 0.25, 1.125, 0.0068359375):
        z = np.tile(ties * np.float32(scale), width // 16).astype(np.float32)
        rows.append(z)
        rows.append(np.nextafter(z, np.float32(np.inf)).astype(np.float32))
        rows.append(np.nextafter(z, np.float32(-np.inf)).astype(np.float32))
    z = rng.standard_normal(width).astype(np.float32); z[7] = np.inf; z[40] = -np.inf; z[100] = np.inf; z[101] = -np.inf; rows.append(z)
    finite = len(rows)
    z = rng.standard_normal(width).astype(np.float32); z[5] = np.nan; z[63] = np.nan; z[64] = np.nan; z[200:232] = np.nan; rows.append(z)
    z = rng.standard_normal(width).astype(np.float32) * 3; z[0] = 9.0; z[1] = np.nan; z[2] = 0.5; z[33] = -np.nan; z[34] = np.inf; rows.append(z)
    return np.ascontiguousarray(np.stack(rows)), finite


@pytest.mark.parametrize("name", ["Q8_0", "Q4_0", "Q4_1", "Q5_0", "Q5_1", "MXFP4", "NVFP4", "TQ1_0", "TQ2_0"])
def test_edge_blocks_of_the_simple_types(gguf, checker, name):
    qtype = inputs.QTYPES[name]
    x, finite = _edge_rows()
    got, want = gguf.quantize_rows(x, qtype), checker.quantize_rows(x, qtype)
    for r in range(x.shape[0]):
        assert np.array_equal(got[r], want[r]), (name, r, "finite" if r < finite else "with NaN")


@pytest.mark.parametrize("name", ["Q8_0", "Q4_0", "Q6_K"])
def test_large_host_calls_go_through_the_pinned_ring_in_ragged_pieces(gguf, checker, name):
    """A host-pointer call of 82 MB is split into five pieces (four of 4096 rows of 1024 and one of 3616) that overlap on two
    streams; every row must still equal the checker's, with and without an importance row, and decode back bit-exactly."""
    qtype = inputs.QTYPES[name]
    rows, cols = 20000, 1024
    x = (np.random.default_rng(23).standard_normal((rows, cols), dtype=np.float32) * np.float32(0.05))
    want = checker.quantize_rows(x, qtype)
    got = gguf.quantize_rows(x, qtype)
    assert np.array_equal(got, want)
    imatrix = np.random.default_rng(24).random(cols, dtype=np.float32) + np.float32(0.1)
    if name != "Q8_0":
        assert np.array_equal(gguf.quantize_rows(x, qtype, imatrix=imatrix), checker.quantize_rows(x, qtype, imatrix=imatrix))
    dec = gguf.dequantize_rows(got, qtype, cols)
    assert np.array_equal(dec.view(np.uint32), checker.dequantize_rows(want, qtype, cols).view(np.uint32))
    # a chunk that starts inside the matrix
    part = gguf.quantize_rows(x[5000:19000], qtype)
    assert np.array_equal(part, want[5000:19000])


def test_bulk_copy_staging_never_ran_out_of_its_wait_limit(gguf):
    """The ternary quantizers stage their input with bulk asynchronous copies whose waits are bounded; a wait that
    gives up is counted on the device.  A pass over a ragged number of blocks must not move the count."""
    import ctypes
    from libgguf_b200._native import lib
    before, count = ctypes.c_uint64(123), ctypes.c_uint64(123)
    assert lib.libgguf_cuda_staging_timeouts(ctypes.byref(before)) == 0
    x = np.random.default_rng(5).standard_normal((1237, 768), dtype=np.float32)
    for name in ("TQ1_0", "TQ2_0", "Q1_0"):
        gguf.quantize_rows(x, inputs.QTYPES[name])
    assert lib.libgguf_cuda_staging_timeouts(ctypes.byref(count)) == 0
    assert count.value == before.value


@pytest.mark.parametrize("name", ["TQ1_0", "TQ2_0", "Q1_0"])
def test_a_staged_copy_that_is_given_up_on_fails_the_call_instead_of_returning_partial_rows(gguf, checker, name):
    """The consumers' wait limit is set to zero polling rounds, so every CTA gives up on its first tile although the
    copy is on its way: the kernel counts it, waits (bounded, full limit) for the copies it has in flight and returns
    without writing its rows.  Nothing hangs or faults, the context stays usable, and the host-pointer call and the
    conversion pipeline must report failure rather than hand back unwritten bytes."""
    import ctypes
    from libgguf_b200._native import lib
    from libgguf_b200.convert import ConversionPipeline
    qtype = inputs.QTYPES[name]
    x = np.random.default_rng(8).standard_normal((257, 1024), dtype=np.float32)
    want = checker.quantize_rows(x, qtype)
    before, after = ctypes.c_uint64(), ctypes.c_uint64()
    assert lib.libgguf_cuda_staging_timeouts(ctypes.byref(before)) == 0
    assert lib.libgguf_cuda_set_staging_wait_limit(0) == 0
    try:
        with pytest.raises(RuntimeError, match="wrote 0 bytes"):
            gguf.quantize_rows(x, qtype)
        assert lib.libgguf_cuda_staging_timeouts(ctypes.byref(after)) == 0
        assert after.value > before.value
        dst = np.zeros(want.size, np.uint8)
        with ConversionPipeline([0], slots=2, chunk_bytes=256 << 10) as pipe:
            with pytest.raises(RuntimeError, match="did not arrive within its wait limit"):
                pipe.quantize([(qtype, x, None, dst)])
    finally:
        assert lib.libgguf_cuda_set_staging_wait_limit(-1) == 0
    # the default limit is back: same device, same context, correct bytes
    np.testing.assert_array_equal(gguf.quantize_rows(x, qtype), want)
    dst = np.zeros(want.size, np.uint8)
    with ConversionPipeline([0], slots=2, chunk_bytes=256 << 10) as pipe:
        pipe.quantize([(qtype, x, None, dst)])
    np.testing.assert_array_equal(dst.reshape(want.shape), want)
    final = ctypes.c_uint64()
    assert lib.libgguf_cuda_staging_timeouts(ctypes.byref(final)) == 0
    # the pipeline's attempt under the zero limit added its own give-ups; the healthy calls added none
    assert final.value >= after.value
