"""The allocation-free quantize entry point (libgguf_cuda_quantize_weighted_rows_static).

Some users of this library cannot allocate GPU memory when they quantize -- they run inside a
framework that owns the whole device through its own pool, under a fixed memory budget, or in a
loop that cannot afford an allocator call -- so the library offers one entry point whose scratch
is a fixed array inside the library.  This test drives it through the C ABI twice in a row and
requires the bytes to equal those of the regular entry point and of the CPU checker both times
(the array is shared and keeps old contents, so the second call is the one that would show stale
data), then checks the refusals.  The file is named so that pytest collects it after every other test."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _quantize(fn_name, x, im, qtype):
    from libgguf_b200._native import lib
    rows, n = x.shape
    rs = lib.libgguf_cuda_row_size(qtype, n)
    out = torch.full((rows, rs), 0xEE, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    st = getattr(lib, fn_name)(x.data_ptr(), im.data_ptr(), out.data_ptr(), qtype, rows, n, stream)
    torch.cuda.synchronize()
    assert st == 0, lib.libgguf_cuda_thread_last_error().decode()
    return out.cpu().numpy()


@pytest.fixture(scope="module")
def checker():
    from oracle import reference
    return reference.load("ref" if reference.available("ref") else "port")


@pytest.mark.parametrize("qtype", [2, 3, 6, 7])
def test_static_scratch_entry_point_matches_regular_entry_point_twice(qtype, checker):
    rng = np.random.default_rng(qtype)
    im = torch.from_numpy((rng.chisquare(4, 1024) / 4).astype(np.float32)).cuda()
    # first call: many rows with large values, so that the shared array is left full of big numbers
    first = torch.from_numpy((rng.standard_normal((300, 1024)) * 50).astype(np.float32)).cuda()
    # second call: fewer rows of small values -- stale scratch would change the weights and the bytes
    second = torch.from_numpy((rng.standard_normal((37, 1024)) * 0.01).astype(np.float32)).cuda()
    for x in (first, second):
        got = _quantize("libgguf_cuda_quantize_weighted_rows_static", x, im, qtype)
        want = _quantize("libgguf_cuda_quantize_f32_rows_on_stream", x, im, qtype)
        np.testing.assert_array_equal(got, want)  # integer bytes: the tolerance of the other parity tests is zero
        np.testing.assert_array_equal(got, checker.quantize_rows(x.cpu().numpy(), qtype, im.cpu().numpy()))


def test_static_scratch_entry_point_refusals():
    from libgguf_b200._native import lib
    limit = lib.libgguf_cuda_quantize_weighted_rows_static_max_rows()
    assert limit == 65536
    x = torch.zeros((4, 64), device="cuda")
    im = torch.ones(64, device="cuda")
    out = torch.zeros(4 * 64, dtype=torch.uint8, device="cuda")
    fn = lib.libgguf_cuda_quantize_weighted_rows_static
    stream = torch.cuda.current_stream().cuda_stream
    # more rows than the built-in array holds (refused before anything is read, so the small buffers are fine)
    assert fn(x.data_ptr(), im.data_ptr(), out.data_ptr(), 2, limit + 1, 64, stream) == 1
    assert b"65536" in lib.libgguf_cuda_thread_last_error()
    # a type whose quantizer needs no scratch is not offered here
    assert fn(x.data_ptr(), im.data_ptr(), out.data_ptr(), 8, 4, 64, stream) == 2
    # the imatrix is what makes the scratch necessary; without it the regular entry point allocates nothing either
    assert fn(x.data_ptr(), None, out.data_ptr(), 2, 4, 64, stream) == 1
    assert fn(x.data_ptr(), im.data_ptr(), out.data_ptr(), 2, 4, 48, stream) == 1
    assert fn(x.data_ptr(), im.data_ptr(), out.data_ptr(), 2, 0, 64, stream) == 0
