import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def ref():
    """The upstream CPU REF backend compiled by oracle/Makefile (skips if it was never built)."""
    from oracle import reference
    if not reference.available("ref"):
        pytest.skip("oracle/_ref/libgguf_ref.so not built (needs the upstream sources: make -C oracle ref)")
    return reference.load("ref")


@pytest.fixture(scope="session")
def port():
    """This repository's plain-C restatement of the upstream algorithms."""
    from oracle import reference
    if not reference.available("port"):
        import subprocess
        subprocess.run(["make", "-C", str(ROOT / "oracle"), "oracle"], check=True, capture_output=True)
    return reference.load("port")


@pytest.fixture(scope="session")
def gguf():
    import libgguf_b200
    return libgguf_b200
