"""Upstream's own callers of the two C ABIs, compiled unmodified from the upstream sources by oracle/Makefile
(`make -C oracle callers`) and linked to libgguf_b200.so:

  oracle/_ref/quantize_gguf_b200   upstream's native converter (csrc/quantize_gguf.cpp) built with its CUDA path
                                   (cuda_converter_context, :1732-1931, the caller of the libgguf_cuda_* functions:
                                   contexts, events, grow-only device and pinned buffers, h2d / d2h, quantize_f32_rows)
  oracle/_ref/_libgguf.so          upstream's CPython extension (csrc/_libgguf_module.cpp; the calls of the
                                   host-pointer functions are at :1731, :1889, :1988, :2086)

Both are test infrastructure.  The converter must write the files upstream's CPU build wrote (SHA-256 of
tests/golden/converter_golden.json), pass its own --verify-cuda-tensors comparison against its CPU quantizers, and the
extension module must return the checker's bytes."""
import hashlib
import importlib.util
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import inputs

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
REF = ROOT / "oracle" / "_ref"
GOLDEN_DIR = Path(__file__).parent / "golden"
sys.path.insert(0, str(GOLDEN_DIR))
import converter_models as cm  # noqa: E402

GOLDEN = json.loads((GOLDEN_DIR / "converter_golden.json").read_text())["entries"]
CONVERTER = REF / "quantize_gguf_b200"
MODULE = REF / "_libgguf.so"


@pytest.fixture(scope="module")
def checker():
    from oracle import reference
    return reference.load("ref" if reference.available("ref") else "port")


@pytest.fixture(scope="module")
def checkpoints(tmp_path_factory):
    root = tmp_path_factory.mktemp("ckpt_upstream")
    paths = {}
    for name, (builder, _) in cm.CASES.items():
        paths[name] = str(root / f"{name}.safetensors")
        cm.write_safetensors(paths[name], builder(), {"format": "pt"})
    return paths


def _run_converter(args):
    return subprocess.run([str(CONVERTER)] + args, capture_output=True, text=True, timeout=600)


@pytest.mark.parametrize("entry", sorted(GOLDEN))
def test_upstream_converter_on_this_library_writes_upstreams_files(checkpoints, entry, tmp_path):
    """--backend cuda with the two-slot pipeline: every quantized tensor goes through libgguf_cuda_* of this library."""
    if not CONVERTER.exists():
        pytest.skip("oracle/_ref/quantize_gguf_b200 not built (make -C oracle callers)")
    name, _ = entry.split("/")
    gold = GOLDEN[entry]
    dst = tmp_path / "out.gguf"
    r = _run_converter(["--src", checkpoints[name], "--dst", str(dst), "--backend", "cuda", "--cuda-fallback", "cpu",
                        "--cuda-pipeline", "1", "--cuda-batch-mb", "1", "--overwrite", "--timings"] + gold["options"])
    assert r.returncode == 0, r.stderr[-2000:]
    data = dst.read_bytes()
    assert len(data) == gold["size"]
    assert hashlib.sha256(data).hexdigest() == gold["sha256"]
    tokens = dict(t.split("=") for line in r.stderr.splitlines() if line.startswith("Timings: ") for t in line.split()[1:])
    if entry.endswith(("/q1_0", "/q5_0", "/q5_1")):   # not in upstream's converter's CUDA type list (quantize_gguf.cpp:1666-1679): CPU path
        assert int(tokens["cuda_tensors"]) == 0
    else:
        assert int(tokens["cuda_tensors"]) > 0 and int(tokens["cuda_chunks"]) > 0, tokens


@pytest.mark.parametrize("name,options", [("flux_bf16", ["--qtype", "Q4_K_M"]), ("wan_f16", ["--qtype", "Q3_K_M", "--policy", "dynamic"]),
                                          ("flux_f32", ["--qtype", "Q6_K"]), ("sd1_f16", ["--qtype", "Q4_K_M"]),
                                          ("cosmos_bf16", ["--qtype", "Q3_K_L"]), ("flux_f32", ["--qtype", "Q2_K"])])
def test_upstream_converter_verifies_this_librarys_bytes_against_its_cpu_quantizers(checkpoints, name, options, tmp_path):
    """--verify-cuda-tensors all (upstream csrc/quantize_gguf.cpp:2176-2181): upstream itself compares every chunk the
    CUDA context returned with its CPU worker pool's bytes and fails on the first difference."""
    if not CONVERTER.exists():
        pytest.skip("oracle/_ref/quantize_gguf_b200 not built (make -C oracle callers)")
    dst = tmp_path / "verified.gguf"
    r = _run_converter(["--src", checkpoints[name], "--dst", str(dst), "--backend", "cuda", "--cuda-fallback", "cpu",
                        "--verify-cuda-tensors", "all", "--overwrite", "--timings"] + options)
    assert r.returncode == 0, r.stderr[-2000:]
    tokens = dict(t.split("=") for line in r.stderr.splitlines() if line.startswith("Timings: ") for t in line.split()[1:])
    assert int(tokens["cuda_verified"]) == int(tokens["cuda_tensors"]) > 0, tokens


# ------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def upstream_module():
    if not MODULE.exists():
        pytest.skip("oracle/_ref/_libgguf.so not built (make -C oracle callers)")
    spec = importlib.util.spec_from_file_location("_libgguf", MODULE)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


@pytest.mark.parametrize("name", sorted(inputs.QTYPES))
def test_upstream_extension_module_returns_the_checkers_bytes(upstream_module, checker, name):
    """quantize_rows_raw / quantize_rows_into_raw / dequantize_rows_raw / dequantize_rows_into_raw of upstream's
    binding, every block type; the kernels of this library run underneath (the launch counter moves)."""
    from libgguf_b200._native import lib
    m = upstream_module
    qtype = inputs.QTYPES[name]
    rows, width = 24, 1024
    x = np.random.default_rng(qtype).standard_normal((rows, width), dtype=np.float32)
    im = inputs.imatrix_for(width, seed=qtype) if m.quantize_requires_imatrix(qtype) else None
    assert bool(m.quantize_requires_imatrix(qtype)) == checker.requires_imatrix(qtype)
    want = checker.quantize_rows(x, qtype, im)
    rs = m.row_size(qtype, width)
    assert rs == want.shape[-1]
    before = lib.libgguf_cuda_kernel_launch_count()
    raw = m.quantize_rows_raw(qtype, x, rows, width, imatrix=im)
    assert lib.libgguf_cuda_kernel_launch_count() > before, "the module did not reach this library's kernels"
    assert isinstance(raw, bytes) and np.array_equal(np.frombuffer(raw, np.uint8).reshape(rows, rs), want)
    out = np.full(rows * rs + 8, 0xCD, np.uint8)
    assert m.quantize_rows_into_raw(qtype, x, out, rows, width, imatrix=im) == rows * rs
    assert np.array_equal(out[:rows * rs].reshape(rows, rs), want) and (out[rows * rs:] == 0xCD).all()
    ref32 = checker.dequantize_rows(want, qtype, width)
    dec = np.frombuffer(m.dequantize_rows_raw(qtype, want, rows, width), np.float32).reshape(rows, width)
    assert np.array_equal(dec.view(np.uint32), ref32.view(np.uint32))
    dst = np.zeros((rows, width), np.float32)
    assert m.dequantize_rows_into_raw(qtype, want, dst, rows, width) == rows * width * 4
    assert np.array_equal(dst.view(np.uint32), ref32.view(np.uint32))


def test_upstream_extension_module_error_behaviour(upstream_module):
    """The binding's own argument checks sit in front of this library (upstream tests/test_python_api_rows.py:163-306
    exercises them through the Python package); what reaches the C ABI must come back as upstream expects."""
    m = upstream_module
    x = np.zeros((2, 256), np.float32)
    with pytest.raises(ValueError, match="unsupported quantization type or row width"):
        m.quantize_rows_raw(12, x, 2, 100)
    with pytest.raises(ValueError, match="unsupported quantization type or row width"):
        m.quantize_rows_raw(15, x, 2, 256)          # Q8_K has no row quantizer
    with pytest.raises(ValueError, match="imatrix is required"):
        m.quantize_rows_raw(16, x, 2, 256)
    with pytest.raises(ValueError, match="src buffer is smaller"):
        m.quantize_rows_raw(12, x, 3, 256)
    assert m.quantize_rows_raw(12, x, 0, 256) == b""
    assert m.type_name(12) == "q4_K" and m.type_size(12) == 144 and m.row_size(12, 100) == 0
    assert len(m.quantize_rows_raw(12, x, 2, 256)) == 288
    m.quantize_free()                                # releases this library's tables and staging buffers
    assert len(m.quantize_rows_raw(18, x, 2, 256)) == 196   # and they come back on the next use
