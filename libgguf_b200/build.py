"""Builds libgguf_b200.so, the C-ABI shared library with the sm_100a kernels, in-tree.

    python libgguf_b200/build.py [--force] [--verbose]

(run it as a script: importing the package needs the library this script produces)

Every translation unit is compiled with
    -gencode arch=compute_100a,code=sm_100a --fmad=false
(IEEE division and square root and no flush-to-zero are nvcc defaults) because the encoded bytes
must match the upstream CPU REF backend, which is built without FMA contraction
(upstream CMakeLists.txt:76-82; upstream's own CUDA targets pass --fmad=false, :274).
Objects are cached under libgguf_b200/_build and rebuilt when a source or header is newer.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT = PKG / "libgguf_b200.so"
OBJ = PKG / "_build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "--fmad=false", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))


def _headers() -> list[Path]:
    return (sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.inc"))
            + sorted((PKG.parent / "include").glob("*.h")))


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    newest_header = max(h.stat().st_mtime for h in _headers())
    nvcc = _nvcc()
    jobs = []
    objects = []
    for src in _sources():
        obj = OBJ / (src.name + ".o")
        objects.append(obj)
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, newest_header)
        if stale:
            cmd = [nvcc, *NVCC_FLAGS, "-x", "cu", "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0 or verbose:
            sys.stderr.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {cmd[-3]}")

    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as pool:
            list(pool.map(run, jobs))
    if jobs or not OUT.exists():
        # -Bsymbolic-functions: calls between this library's own exported functions stay inside it even when a
        # program also links the upstream CPU library, which exports the same seven host-pointer names
        link = [nvcc, "-shared", "-o", str(OUT), *map(str, objects), "-cudart", "static", "-lpthread",
                "-Xlinker", "-Bsymbolic-functions"]
        run(link)
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args()
    print(build(force=args.force, verbose=args.verbose))
