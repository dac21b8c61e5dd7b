"""Regenerates tests/golden/converter_golden.json: SHA-256 of the files upstream's native converter writes (CPU
backend) for the synthetic checkpoints of converter_models.py.

Needs the upstream converter built by `make -C oracle converter` (oracle/_ref/quantize_gguf_ref, compiled from the
upstream sources).  Run from the repository root:  python tests/golden/make_converter_golden.py"""
import hashlib
import json
import os
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
import converter_models as cm  # noqa: E402

CONVERTER = HERE.parents[1] / "oracle" / "_ref" / "quantize_gguf_ref"


def main():
    out = {"note": "sha256 of upstream libgguf_quantize_gguf --backend cpu output per synthetic checkpoint and option set", "entries": {}}
    with tempfile.TemporaryDirectory() as tmp:
        for name, (builder, cases) in cm.CASES.items():
            src = os.path.join(tmp, name + ".safetensors")
            cm.write_safetensors(src, builder(), {"format": "pt"})
            src_hash = hashlib.sha256(open(src, "rb").read()).hexdigest()
            for case, opts in cases:
                dst = os.path.join(tmp, f"{name}-{case}.gguf")
                r = subprocess.run([str(CONVERTER), "--src", src, "--dst", dst, "--backend", "cpu", "--overwrite"] + opts,
                                   capture_output=True, text=True, check=True)
                data = open(dst, "rb").read()
                out["entries"][f"{name}/{case}"] = {"options": opts, "source_sha256": src_hash, "size": len(data),
                                                   "sha256": hashlib.sha256(data).hexdigest(),
                                                   "summary": r.stdout.strip().splitlines()[1:]}
    (HERE / "converter_golden.json").write_text(json.dumps(out, indent=1) + "\n")
    print(len(out["entries"]), "entries")


if __name__ == "__main__":
    main()
