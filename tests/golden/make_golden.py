#!/usr/bin/env python3
"""Regenerates the golden fixtures of tests/golden/ from the upstream reference.

    python tests/golden/make_golden.py [--upstream /path/to/upstream/checkout]

Writes
  upstream_manifest.json  the 70 frozen SHA-256 entries of upstream tests/golden/manifest.json
                          (qtype, shape, pattern, byte count, hash), copied as data so the pin
                          travels without the upstream checkout;
  golden.json             SHA-256 of encoded bytes and of the decoded fp32 bytes for every
                          quantized type x pattern (with and without importance weights),
                          produced by running the upstream CPU REF backend
                          (oracle/_ref/libgguf_ref.so, built by oracle/Makefile) on the seeded
                          inputs of tests/inputs.py.
The tests check the oracle and the CUDA path against both files.
"""
from __future__ import annotations

import argparse
import os
import hashlib
import json
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import inputs  # noqa: E402
from oracle import reference  # noqa: E402

ROWS, WIDTH = 4, 1024


def sha(a) -> str:
    return hashlib.sha256(a.tobytes()).hexdigest()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--upstream", default=os.environ.get("LIBGGUF_UPSTREAM_ROOT"),
                    help="the upstream libgguf checkout (default: $LIBGGUF_UPSTREAM_ROOT)")
    args = ap.parse_args()
    if not args.upstream:
        ap.error("--upstream PATH (or LIBGGUF_UPSTREAM_ROOT) is required")
    manifest = json.loads((Path(args.upstream) / "tests/golden/manifest.json").read_text())
    entries = [{k: e[k] for k in ("qtype", "shape", "pattern", "encoded_nbytes", "encoded_sha256")} for e in manifest["entries"]]
    (HERE / "upstream_manifest.json").write_text(json.dumps({"source": "upstream tests/golden/manifest.json", "entries": entries}, indent=1) + "\n")

    ref = reference.load("ref")
    out = []
    for name, qtype in inputs.QTYPES.items():
        for pattern in inputs.PATTERNS:
            x = inputs.pattern_rows(pattern, ROWS, WIDTH, seed=qtype * 1009 + sum(pattern.encode()))
            for weighted in (False, True):
                im = inputs.imatrix_for(WIDTH, seed=qtype) if weighted else None
                enc = ref.quantize_rows(x, qtype, im)
                dec = ref.dequantize_rows(enc, qtype, WIDTH)
                out.append({"qtype": name, "pattern": pattern, "weighted": weighted, "rows": ROWS, "width": WIDTH,
                            "encoded_sha256": sha(enc), "decoded_sha256": sha(dec)})
    (HERE / "golden.json").write_text(json.dumps({"generator": "tests/golden/make_golden.py", "entries": out}, indent=1) + "\n")
    print(f"wrote {len(entries)} upstream pins and {len(out)} golden entries")


if __name__ == "__main__":
    main()
