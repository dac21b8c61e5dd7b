"""Checked mode (LIBGGUF_B200_CHECKED=1): the host-pointer calls run with guard bands around the device bytes their
kernels may touch.  Ragged shapes of every block type go through in a child process (the mode is read when the
library is loaded): the results must equal the CPU checker's (a read past the end of the input would pull NaN bytes
in) and no guard byte may have changed (a write outside the output).  This is the stand-in for a memory checker,
which cannot be run where these tests run."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]

CHILD = r"""
import ctypes, sys
import numpy as np
sys.path.insert(0, {root!r}); sys.path.insert(0, {tests!r})
import inputs
import libgguf_b200 as g
from libgguf_b200._native import lib
from oracle import reference
chk = reference.load("ref" if reference.available("ref") else "port")
count = ctypes.c_uint64(99)
assert lib.libgguf_cuda_checked_violations(ctypes.byref(count)) == 0 and count.value == 0, "checked mode is off"
rng = np.random.default_rng(17)
cases = 0
for name, qtype in sorted(inputs.QTYPES.items()):
    block = inputs.block_size(name)
    for rows, width in ((1, block), (3, 3 * block), (5, 7 * block), (33, block), (130, 2 * block), (17, 11 * block)):
        x = rng.standard_normal((rows, width), dtype=np.float32)
        im = inputs.imatrix_for(width, seed=qtype) if chk.requires_imatrix(qtype) else None
        want = chk.quantize_rows(x, qtype, im)
        for repeat in range(3):   # a race would show as a difference between repeated runs
            got = g.quantize_rows(x, qtype, im)
            assert np.array_equal(got, want), (name, rows, width, "quantize", repeat)
        dec = g.dequantize_rows(want, qtype, width)
        assert np.array_equal(dec.view(np.uint32), chk.dequantize_rows(want, qtype, width).view(np.uint32)), (name, rows, width, "decode")
        cases += 1
assert lib.libgguf_cuda_checked_violations(ctypes.byref(count)) == 0
print("cases", cases, "violations", count.value)
assert count.value == 0
"""


def test_ragged_shapes_in_checked_mode_touch_nothing_outside_their_buffers():
    env = dict(os.environ, LIBGGUF_B200_CHECKED="1")
    r = subprocess.run([sys.executable, "-c", CHILD.format(root=str(ROOT), tests=str(ROOT / "tests"))], env=env,
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "violations 0" in r.stdout


def test_checked_mode_is_off_by_default():
    import ctypes
    from libgguf_b200._native import lib
    if os.environ.get("LIBGGUF_B200_CHECKED", "0") not in ("", "0"):
        pytest.skip("the test process itself runs in checked mode")
    count = ctypes.c_uint64(5)
    assert lib.libgguf_cuda_checked_violations(ctypes.byref(count)) == 2 and count.value == 0
