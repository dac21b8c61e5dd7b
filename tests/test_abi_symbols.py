"""The C-ABI shared library loads and exports every function the public headers declare
(no compute calls, so no GPU needed)."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def declared_functions(header: Path) -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
    text = re.sub(r"//.*", "", text)
    return re.findall(r"\b(libgguf_[a-z0-9_]+)\s*\(", text)


def test_library_exports_every_declared_symbol():
    from libgguf_b200 import _native
    lib = ctypes.CDLL(str(_native.LIB_PATH))
    names = []
    for header in sorted((ROOT / "include").glob("*.h")):
        names += declared_functions(header)
    assert len(set(names)) >= 7 + 30
    missing = [n for n in sorted(set(names)) if not hasattr(lib, n)]
    assert not missing, missing


def test_binding_table_covers_the_headers():
    from libgguf_b200 import _native
    bound = set(_native.HOST_ABI) | set(_native.NATIVE_ABI)
    declared = set()
    for header in sorted((ROOT / "include").glob("*.h")):
        declared |= set(declared_functions(header))
    assert declared == bound


def test_type_queries_need_no_device():
    from libgguf_b200._native import lib
    assert lib.libgguf_cuda_qtype_supported(12) == 1
    assert lib.libgguf_cuda_qtype_supported(0) == 0
    assert lib.libgguf_cuda_qtype_needs_imatrix(16) == 1
    assert lib.libgguf_cuda_block_size(12) == 256
    assert lib.libgguf_cuda_row_size(12, 4096) == 2304
    assert lib.libgguf_cuda_dequantize_qtype_supported(30) == 1
    assert lib.libgguf_cuda_dequantize_block_size(30) == 1
    assert lib.libgguf_cuda_dequantize_row_size(30, 10) == 20
    assert lib.libgguf_cuda_dequantize_row_size(14, 256) == 210
    assert lib.libgguf_cuda_last_error(None) == b"libgguf CUDA context is null"


def test_host_copy_pool_copies_every_byte():
    """The copy pool behind the host-pointer calls (no device involved): large, odd-sized and back-to-back
    copies arrive intact and touch nothing past their end."""
    import numpy as np
    from libgguf_b200 import _native
    lib = ctypes.CDLL(str(_native.LIB_PATH))
    lib.libgguf_cuda_host_copy.restype = None
    lib.libgguf_cuda_host_copy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]
    rng = np.random.default_rng(3)
    src = rng.integers(0, 256, size=48 << 20, dtype=np.uint8)
    for offset, size in [(0, 48 << 20), (1, (33 << 20) + 12345), (7, (2 << 20) + 1), (3, 4096), (0, 0)] + [(i, (3 << 20) + 7777 * i) for i in range(1, 40)]:
        dst = np.full(size + 64, 0xA5, dtype=np.uint8)
        lib.libgguf_cuda_host_copy(dst.ctypes.data, src.ctypes.data + offset, size)
        assert np.array_equal(dst[:size], src[offset:offset + size])
        assert (dst[size:] == 0xA5).all()


def test_public_header_compiles_as_c_and_keeps_upstreams_enums(tmp_path):
    """A C program written against upstream's include/libgguf.h (:16-100: ggml_type, ggml_prec, ggml_ftype) compiles
    against this repository's header, links to the library, and sees the same enum values."""
    import shutil
    import subprocess
    from libgguf_b200 import _native
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        import pytest
        pytest.skip("no C compiler")
    src = tmp_path / "t.c"
    src.write_text('''
#include <stdio.h>
#include "libgguf.h"
int main(void) {
    enum ggml_ftype f = GGML_FTYPE_MOSTLY_Q4_K;
    enum ggml_prec p = GGML_PREC_F32;
    printf("%d %d %d %d %d %zu %s\\n", (int)f, (int)p, (int)GGML_FTYPE_UNKNOWN, (int)GGML_FTYPE_MOSTLY_Q1_0, (int)GGML_TYPE_COUNT,
           libgguf_row_size(GGML_TYPE_Q4_K, 4096), libgguf_type_name(GGML_TYPE_IQ2_XXS));
    return 0;
}
''')
    exe = tmp_path / "t"
    lib_dir = _native.LIB_PATH.parent
    subprocess.run([cc, "-std=c99", "-Wall", "-Werror", "-I", str(ROOT / "include"), str(src), "-o", str(exe),
                    "-L", str(lib_dir), f"-l:{_native.LIB_PATH.name}", f"-Wl,-rpath,{lib_dir}"], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    assert out == ["12", "10", "-1", "27", "42", "2304", "iq2_xxs"]
