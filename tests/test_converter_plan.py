"""The converter front end without a GPU: planning, GGUF header and summary against the files upstream's native
converter wrote for the same synthetic checkpoints (tests/golden/converter_golden.json), plus the reader."""
import hashlib
import json
import sys
from pathlib import Path

import numpy as np
import pytest

GOLDEN_DIR = Path(__file__).parent / "golden"
sys.path.insert(0, str(GOLDEN_DIR))
import converter_models as cm  # noqa: E402

from libgguf_b200 import GGMLQuantizationType as Q  # noqa: E402
from libgguf_b200 import quantize_gguf as qg  # noqa: E402
from libgguf_b200 import row_size  # noqa: E402
from libgguf_b200.gguf_file import TensorInfo, header_bytes, pad_to, read_gguf  # noqa: E402

GOLDEN = json.loads((GOLDEN_DIR / "converter_golden.json").read_text())["entries"]


@pytest.fixture(scope="module")
def checkpoints(tmp_path_factory):
    root = tmp_path_factory.mktemp("ckpt")
    paths = {}
    for name, (builder, _) in cm.CASES.items():
        paths[name] = str(root / f"{name}.safetensors")
        cm.write_safetensors(paths[name], builder(), {"format": "pt"})
    return paths


@pytest.mark.parametrize("entry", sorted(GOLDEN))
def test_plan_and_summary_match_upstream(checkpoints, entry, tmp_path):
    name, _ = entry.split("/")
    gold = GOLDEN[entry]
    assert hashlib.sha256(open(checkpoints[name], "rb").read()).hexdigest() == gold["source_sha256"]
    options = qg.parse_args(["--src", checkpoints[name], "--dst", str(tmp_path / "o.gguf")] + gold["options"])
    _, _, _, kv, plans, result = qg.plan_file(options)
    head = header_bytes(kv, [TensorInfo(p.key, tuple(p.write_shape), int(Q[p.qtype]), p.nbytes) for p in plans])
    assert pad_to(len(head)) + sum(pad_to(p.nbytes) for p in plans) == gold["size"]
    assert qg.summary_lines(result)[1:] == gold["summary"]


def test_pattern_matcher():
    assert qg.fnmatch_case("*attn_v.weight*", "blk.3.attn_v.weight")
    assert qg.fnmatch_case("double_layers.*.mlp?.c_proj.weight", "double_layers.12.mlpX.c_proj.weight")
    assert not qg.fnmatch_case("double_layers.*.mlp?.c_proj.weight", "double_layers.12.mlp.c_proj.weight")
    assert qg.fnmatch_case("**", "") and qg.fnmatch_case("a*b*c", "a__b__bc") and not qg.fnmatch_case("a*b", "a__c")
    assert not qg.fnmatch_case("[ab]", "a") and qg.fnmatch_case("[ab]", "[ab]")


def test_rejections(tmp_path, checkpoints):
    src = checkpoints["flux_bf16"]
    for argv, message in [(["--qtype", "Q8_K"], "Q8_K output is not supported"), (["--qtype", "F16"], "unsupported direct quantization type"),
                          (["--qtype", "NVFP4"], "non-Q/K quantization families"), (["--qtype", "Q4_K_L"], "unsupported output file type")]:
        with pytest.raises(qg.ConversionError, match=message):
            qg.plan_file(qg.parse_args(["--src", src, "--dst", str(tmp_path / "x.gguf")] + argv))
    with pytest.raises(qg.ConversionError, match="CPU backend requested"):
        qg.parse_args(["--src", src, "--backend", "cpu"])
    accepted = qg.parse_args(["--src", src, "--imatrix", "x.dat", "--threads", "4", "--scratch-bytes", "1024", "--cuda-batch-mb", "64",
                              "--cuda-pipeline", "0", "--verify-cuda-tensors", "all", "--seed", "3", "--timings"])
    assert accepted.chunk_bytes == 64 << 20 and accepted.timings
    with pytest.raises(qg.ConversionError, match="unsupported GGML tensor type"):
        qg.parse_args(["--src", src, "--tensor-type", "*=Q4_K_L"])
    unknown = str(tmp_path / "unknown.safetensors")
    cm.write_safetensors(unknown, [("a.weight", "F32", np.zeros((4, 256), np.float32))])
    with pytest.raises(qg.ConversionError, match="Unknown model architecture"):
        qg.plan_file(qg.parse_args(["--src", unknown, "--dst", str(tmp_path / "x.gguf")]))
    existing = tmp_path / "exists.gguf"
    existing.write_bytes(b"x")
    with pytest.raises(qg.ConversionError, match="Output exists"):
        qg.plan_file(qg.parse_args(["--src", src, "--dst", str(existing)]))
    truncated = str(tmp_path / "trunc.safetensors")
    Path(truncated).write_bytes(open(src, "rb").read()[:-10])
    with pytest.raises(qg.ConversionError, match="exceeds file size"):
        qg.plan_file(qg.parse_args(["--src", truncated, "--dst", str(tmp_path / "x.gguf")]))


def test_llama_checkpoints_get_the_q4_k_m_mix(tmp_path):
    src = str(tmp_path / "llama.safetensors")
    cm.write_safetensors(src, cm.llama_like(layers=32))
    _, _, model, kv, plans, result = qg.plan_file(qg.parse_args(["--src", src, "--dst", str(tmp_path / "l.gguf"), "--qtype", "Q4_K_M"]))
    assert model.arch == "llama" and kv[0][2] == "llama"
    by_key = {p.key: p.qtype for p in plans}
    assert by_key["lm_head.weight"] == "Q6_K" and by_key["model.embed_tokens.weight"] == "Q4_K" and by_key["model.norm.weight"] == "F32"
    more = [i for i in range(32) if by_key[f"model.layers.{i}.self_attn.v_proj.weight"] == "Q6_K"]
    assert more == [i for i in range(32) if by_key[f"model.layers.{i}.mlp.down_proj.weight"] == "Q6_K"]
    assert len(more) == 16 and more[:5] == [0, 1, 2, 3, 6]
    assert all(by_key[f"model.layers.{i}.self_attn.q_proj.weight"] == "Q4_K" for i in range(32))
    assert qg.plan_file(qg.parse_args(["--src", src, "--dst", str(tmp_path / "l.gguf"), "--qtype", "IQ4_XS"]))[1] == "IQ4_XS"


def test_reader_round_trips_the_writer(tmp_path):
    infos = [TensorInfo("a.weight", (4, 256), int(Q.Q4_K), 4 * 144), TensorInfo("b", (7,), int(Q.F32), 28), TensorInfo("s", (), int(Q.F32), 4)]
    kv = [("general.architecture", 8, "flux"), ("general.file_type", 4, 15), ("comfy.gguf.orig_shape.a.weight", 9, (11, [2, 2, 256])),
          ("names", 9, (8, ["x", "yz"])), ("general.alignment", 4, 32)]
    head = header_bytes(kv, infos)
    path = tmp_path / "t.gguf"
    payload = [np.arange(i.nbytes, dtype=np.uint8) for i in infos]
    with open(path, "wb") as f:
        f.write(head + b"\0" * (pad_to(len(head)) - len(head)))
        for p in payload:
            f.write(p.tobytes() + b"\0" * (pad_to(p.size) - p.size))
    g = read_gguf(str(path), row_size)
    assert g.metadata["general.architecture"] == "flux" and g.metadata["comfy.gguf.orig_shape.a.weight"] == [2, 2, 256]
    assert g.metadata["names"] == ["x", "yz"]
    assert [t.shape for t in g.tensors.values()] == [(4, 256), (7,), ()]
    for info, p in zip(infos, payload):
        assert np.array_equal(g.tensor_bytes(info.name), p)
    assert [t.nbytes for t in read_gguf(str(path)).tensors.values()] == [576, 32, 32]  # without sizes: distance to the next tensor
    with pytest.raises(ValueError):
        (tmp_path / "bad.gguf").write_bytes(b"GGUX" + bytes(40))
        read_gguf(str(tmp_path / "bad.gguf"))


def test_gpu_selection_by_count_list_and_environment(monkeypatch):
    """--gpus N, --gpus a,b,c and LIBGGUF_CUDA_DEVICES (default: every visible device)."""
    import pytest
    from libgguf_b200 import quantize_gguf as qg
    base = ["--src", "x.safetensors", "--qtype", "Q4_K_M"]
    monkeypatch.delenv("LIBGGUF_CUDA_DEVICES", raising=False)
    o = qg.parse_args(base)
    assert (o.gpus, o.devices) == (0, ()) and qg.resolve_devices(o.gpus, o.devices, 8) == list(range(8))
    o = qg.parse_args(base + ["--gpus", "3"])
    assert qg.resolve_devices(o.gpus, o.devices, 8) == [0, 1, 2]
    o = qg.parse_args(base + ["--gpus", "0,2,5"])
    assert qg.resolve_devices(o.gpus, o.devices, 8) == [0, 2, 5]
    o = qg.parse_args(base + ["--gpus", "4,"])
    assert qg.resolve_devices(o.gpus, o.devices, 8) == [4]
    monkeypatch.setenv("LIBGGUF_CUDA_DEVICES", "1,3")
    o = qg.parse_args(base)
    assert qg.resolve_devices(o.gpus, o.devices, 4) == [1, 3]
    o = qg.parse_args(base + ["--gpus", "2"])          # the flag wins over the environment
    assert qg.resolve_devices(o.gpus, o.devices, 4) == [0, 1]
    for bad in ("a", "1,1", "-2", "0,-1"):
        with pytest.raises(qg.ConversionError, match="invalid GPU selection"):
            qg.parse_args(base + ["--gpus", bad])
    with pytest.raises(qg.ConversionError, match="only 2 device"):
        qg.resolve_devices(0, (0, 2), 2)
    with pytest.raises(qg.ConversionError, match="only 2 device"):
        qg.resolve_devices(4, (), 2)
