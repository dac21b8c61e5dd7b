"""The whole converter on the GPU: the files it writes must be byte-identical to the ones upstream's native
converter wrote on the CPU for the same synthetic checkpoints (tests/golden/converter_golden.json)."""
import hashlib
import json
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
GOLDEN_DIR = Path(__file__).parent / "golden"
sys.path.insert(0, str(GOLDEN_DIR))
import converter_models as cm  # noqa: E402

GOLDEN = json.loads((GOLDEN_DIR / "converter_golden.json").read_text())["entries"]
UPSTREAM_CONVERTER = Path(__file__).parents[1] / "oracle" / "_ref" / "quantize_gguf_ref"


@pytest.fixture(scope="module")
def checker():
    from oracle import reference
    return reference.load("ref" if reference.available("ref") else "port")


@pytest.fixture(scope="module")
def checkpoints(tmp_path_factory):
    root = tmp_path_factory.mktemp("ckpt")
    paths = {}
    for name, (builder, _) in cm.CASES.items():
        paths[name] = str(root / f"{name}.safetensors")
        cm.write_safetensors(paths[name], builder(), {"format": "pt"})
    return paths


@pytest.mark.parametrize("entry", sorted(GOLDEN))
def test_files_equal_upstreams(gguf, checkpoints, entry, tmp_path, capsys):
    from libgguf_b200 import quantize_gguf as qg
    name, _ = entry.split("/")
    gold = GOLDEN[entry]
    dst = tmp_path / "out.gguf"
    assert qg.main(["--src", checkpoints[name], "--dst", str(dst), "--chunk-mb", "1", "--batch-mb", "1"] + gold["options"]) == 0
    data = dst.read_bytes()
    assert len(data) == gold["size"]
    assert hashlib.sha256(data).hexdigest() == gold["sha256"]
    assert capsys.readouterr().out.strip().splitlines()[1:] == gold["summary"]


def test_load_time_decode_of_a_file_upstream_wrote(gguf, checker, checkpoints, tmp_path):
    """A GGUF file written by upstream's own converter (CPU backend): every tensor read with this repository's reader
    and decoded on the GPU must equal the checker's decode of the stored bytes (fp32 bits; fp16 = its RNE rounding)."""
    import subprocess
    torch = pytest.importorskip("torch")
    if not UPSTREAM_CONVERTER.exists():
        pytest.skip("oracle/_ref/quantize_gguf_ref not built (make -C oracle converter)")
    from libgguf_b200.gguf_file import read_gguf
    from libgguf_b200.libgguf_cuda import load
    for name, options in (("flux_bf16", ["--qtype", "Q4_K_M"]), ("wan_f16", ["--qtype", "Q3_K_M", "--policy", "dynamic"])):
        if name not in checkpoints:
            name = sorted(checkpoints)[0]
        dst = str(tmp_path / f"{name}-upstream.gguf")
        subprocess.run([str(UPSTREAM_CONVERTER), "--src", checkpoints[name], "--dst", dst, "--backend", "cpu", "--overwrite"] + options,
                       check=True, capture_output=True)
        g = read_gguf(dst, gguf.row_size)
        decoded = 0
        for tname, info in g.tensors.items():
            raw = np.array(g.tensor_bytes(tname))
            n = info.shape[-1]
            if info.qtype == 0:
                want = raw.view(np.float32)
            elif info.qtype == 1:
                want = raw.view(np.float16).astype(np.float32)
            elif info.qtype == 30:
                want = (raw.view(np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)
            else:
                want = checker.dequantize_rows(raw.reshape(-1, gguf.row_size(info.qtype, n)), info.qtype, n)
                decoded += 1
            t = load.load_tensor(g, tname, device="cuda", dtype=torch.float32)
            assert tuple(t.shape) == info.shape
            assert np.array_equal(t.cpu().numpy().reshape(-1).view(np.uint32), np.ascontiguousarray(want, np.float32).reshape(-1).view(np.uint32)), tname
            h = load.load_tensor(g, tname, device="cuda", dtype=torch.float16)
            assert torch.equal(h.cpu().reshape(-1).view(torch.int16),
                               torch.from_numpy(np.ascontiguousarray(want, np.float32).reshape(-1)).to(torch.float16).view(torch.int16)), tname
        assert decoded > 0


def test_llama_checkpoint_and_load_time_decode(gguf, checker, tmp_path):
    """Extension types end to end: a Llama-style checkpoint to IQ4_XS / Q4_K_M, read back, decoded on the GPU and
    compared with the checker's decode of the same stored bytes."""
    torch = pytest.importorskip("torch")
    from libgguf_b200 import quantize_gguf as qg
    from libgguf_b200.gguf_file import read_gguf
    from libgguf_b200.libgguf_cuda import load
    src = str(tmp_path / "llama.safetensors")
    cm.write_safetensors(src, cm.llama_like(layers=8))
    for qtype in ("Q4_K_M", "IQ4_XS", "IQ2_XXS"):
        dst = str(tmp_path / f"llama-{qtype}.gguf")
        assert qg.main(["--src", src, "--dst", dst, "--qtype", qtype, "--gpus", "1"]) == 0
        g = read_gguf(dst, gguf.row_size)
        assert g.metadata["general.architecture"] == "llama"
        for name in ("model.layers.3.mlp.down_proj.weight", "lm_head.weight", "model.norm.weight"):
            info = g.tensors[name]
            t = load.load_tensor(g, name, device="cuda", dtype=torch.float32)
            assert tuple(t.shape) == info.shape
            want = checker.dequantize_rows(np.array(g.tensor_bytes(name)).reshape(-1, gguf.row_size(info.qtype, info.shape[-1])), info.qtype,
                                           info.shape[-1]) if info.qtype not in (0,) else np.array(g.tensor_bytes(name)).view(np.float32)
            assert np.array_equal(t.cpu().numpy().reshape(-1).view(np.uint32), np.asarray(want, dtype=np.float32).reshape(-1).view(np.uint32))
        half = load.load_tensor(g, "lm_head.weight", device="cuda", dtype=torch.float16)
        assert half.dtype == torch.float16 and tuple(half.shape) == (512, 256)


def test_timings_line_has_upstreams_tokens(gguf, tmp_path, capsys):
    """--timings prints the token line upstream's benchmark scripts parse (csrc/quantize_gguf.cpp:2527-2547)."""
    import re
    from libgguf_b200 import quantize_gguf as qg
    src = str(tmp_path / "llama.safetensors")
    cm.write_safetensors(src, cm.llama_like(layers=2))
    assert qg.main(["--src", src, "--dst", str(tmp_path / "t.gguf"), "--qtype", "Q4_K_M", "--gpus", "1", "--timings"]) == 0
    line = [l for l in capsys.readouterr().err.splitlines() if l.startswith("Timings: ")]
    assert len(line) == 1
    tokens = dict(t.split("=") for t in line[0].split()[1:])
    assert list(tokens) == ["total", "metadata", "read", "cpu_convert", "h2d", "cuda_quant", "d2h", "write", "tensors", "cuda_tensors",
                            "cuda_verified", "cuda_chunks", "threads", "scratch", "cuda_vram", "cuda_pipeline", "cuda_max_input",
                            "cuda_max_output"]
    assert all(re.fullmatch(r"\d+\.\d{3}s", tokens[k]) for k in list(tokens)[:8])
    assert int(tokens["tensors"]) >= int(tokens["cuda_tensors"]) > 0 and int(tokens["cuda_chunks"]) > 0


def test_tensor_cut_into_pieces_keeps_whole_tensor_importance_weights(gguf, checker, tmp_path):
    """IQ2_XXS needs importance weights; without an imatrix file they are the column sums of squares of the WHOLE tensor
    (upstream compute_auto_imatrix, csrc/_libgguf_module.cpp:1210-1242).  A small --batch-mb cuts the 768-row tensors into
    two pieces: the file must be byte-identical to the uncut conversion, and the cut tensor's bytes equal the checker's."""
    from libgguf_b200 import quantize_gguf as qg
    from libgguf_b200.gguf_file import read_gguf
    tensors = cm.llama_like(layers=2)
    src = str(tmp_path / "llama.safetensors")
    cm.write_safetensors(src, tensors)
    cut, whole = str(tmp_path / "cut.gguf"), str(tmp_path / "whole.gguf")
    assert qg.main(["--src", src, "--dst", cut, "--qtype", "IQ2_XXS", "--gpus", "1", "--batch-mb", "1", "--chunk-mb", "1"]) == 0
    assert qg.main(["--src", src, "--dst", whole, "--qtype", "IQ2_XXS", "--gpus", "1"]) == 0
    assert Path(cut).read_bytes() == Path(whole).read_bytes()
    g = read_gguf(cut, gguf.row_size)
    name = "model.layers.1.mlp.gate_proj.weight"
    values = dict((n, v) for n, _, v in tensors)[name]
    bf16 = (values.astype(np.float32).view(np.uint32) >> 16).astype(np.uint32) << 16
    widened = bf16.view(np.float32)
    info = g.tensors[name]
    assert info.qtype == 16 and info.shape == (768, 256)
    np.testing.assert_array_equal(np.array(g.tensor_bytes(name)).reshape(768, -1), checker.quantize_rows(widened, 16))


def test_rank_slices_of_a_tensor_use_the_whole_tensors_importance_weights(gguf, checker):
    """One process per GPU: each rank encodes a row range.  For a type that needs importance weights and has none, every
    rank derives them from the whole tensor, so the assembled bytes equal the single-call result."""
    from libgguf_b200.convert import ConversionPipeline, rank_batch
    x = np.random.default_rng(12).standard_normal((900, 512), dtype=np.float32)
    want = checker.quantize_rows(x, 19)   # IQ1_S, weights = column sums of squares over all 900 rows
    dst = np.zeros(want.size, np.uint8)
    for rank in range(2):
        batch = rank_batch([(19, x, None, dst)], 2, rank, chunk_bytes=256 << 10)
        assert batch and all(im is not None for _, _, im, _ in batch)
        with ConversionPipeline([0], slots=2, chunk_bytes=128 << 10) as pipe:
            pipe.quantize(batch)
    np.testing.assert_array_equal(dst.reshape(want.shape), want)


def test_a_row_wider_than_the_batch_still_converts_and_failures_leave_no_file(gguf, checker, tmp_path):
    from libgguf_b200 import quantize_gguf as qg
    from libgguf_b200.gguf_file import read_gguf
    rng = np.random.default_rng(3)
    wide = (rng.standard_normal((3, 131072)) * 0.05).astype(np.float32)    # 512 KiB per row, batch arena 256 KiB
    src = str(tmp_path / "wide.safetensors")
    cm.write_safetensors(src, [("model.layers.0.mlp.down_proj.weight", "F32", wide), ("model.norm.weight", "F32", wide[0, :256]),
                               ("model.layers.0.self_attn.q_proj.weight", "F32", np.ascontiguousarray(wide[:, :256]))])
    dst = str(tmp_path / "wide.gguf")
    assert qg.main(["--src", src, "--dst", dst, "--qtype", "Q8_0", "--gpus", "1", "--batch-mb", "1"]) == 0
    g = read_gguf(dst, gguf.row_size)
    name = "model.layers.0.mlp.down_proj.weight"
    np.testing.assert_array_equal(np.array(g.tensor_bytes(name)).reshape(3, -1), checker.quantize_rows(wide, 8))
    # a conversion that fails half way removes what it had written
    broken = str(tmp_path / "broken.gguf")
    import libgguf_b200.convert as conv

    class Failing(conv.ConversionPipeline):
        def quantize(self, tensors):
            raise RuntimeError("injected")

    original = conv.ConversionPipeline
    conv.ConversionPipeline = Failing
    try:
        with pytest.raises(RuntimeError, match="injected"):
            qg.convert(qg.parse_args(["--src", src, "--dst", broken, "--qtype", "Q8_0", "--gpus", "1"]))
    finally:
        conv.ConversionPipeline = original
    assert not Path(broken).exists()


def test_a_full_file_system_is_an_error_before_anything_is_written(tmp_path, monkeypatch):
    """The output is filled through a shared mapping, where running out of blocks would be a fault inside a copy; the
    converter therefore checks the free space first and reports ENOSPC as an OSError, leaving no file."""
    import errno
    import os
    from libgguf_b200 import quantize_gguf as qg
    rng = np.random.default_rng(5)
    w = (rng.standard_normal((64, 1024)) * 0.05).astype(np.float32)
    src = str(tmp_path / "m.safetensors")
    cm.write_safetensors(src, [("model.layers.0.self_attn.q_proj.weight", "F32", w), ("model.layers.0.mlp.down_proj.weight", "F32", w),
                               ("model.norm.weight", "F32", w[0, :256])])
    dst = str(tmp_path / "full.gguf")
    real = os.fstatvfs

    class NoRoom:
        def __init__(self, st):
            self.f_blocks, self.f_frsize, self.f_bavail = st.f_blocks, st.f_frsize, 0

    monkeypatch.setattr(os, "fstatvfs", lambda fd: NoRoom(real(fd)))
    with pytest.raises(OSError) as caught:
        qg.convert(qg.parse_args(["--src", src, "--dst", dst, "--qtype", "Q8_0", "--gpus", "1"]))
    assert caught.value.errno == errno.ENOSPC
    assert not Path(dst).exists()
    monkeypatch.undo()
    assert qg.main(["--src", src, "--dst", dst, "--qtype", "Q8_0", "--gpus", "1"]) == 0 and Path(dst).stat().st_size > w.size
