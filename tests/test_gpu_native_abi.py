"""Device-pointer C ABI and the Torch entry points (upstream
tests/backends/libgguf_cuda/test_cuda_native_dequantize.py, test_cuda_quantize.py,
test_cuda_dequantize.py)."""
import ctypes

import numpy as np
import pytest

import inputs

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def checker():
    from oracle import reference
    if reference.available("ref"):
        return reference.load("ref")
    return reference.load("port")


@pytest.fixture(scope="module")
def ops():
    from libgguf_b200.libgguf_cuda import ops
    return ops


@pytest.mark.parametrize("name", sorted(inputs.QTYPES))
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_dequantize_dtypes(ops, checker, name, dtype):
    """fp32 bit-exact; fp16 / bf16 equal to the correctly rounded fp32 decode."""
    qtype = inputs.QTYPES[name]
    x = (np.random.default_rng(11).standard_normal((40, 1024), dtype=np.float32))
    try:
        enc = checker.quantize_rows(x, qtype)
    except Exception:
        pytest.skip("checker cannot encode this type")
    want = torch.from_numpy(checker.dequantize_rows(enc, qtype, 1024))
    got = ops.dequantize(torch.from_numpy(enc).cuda().reshape(-1), qtype, 40, 1024, dtype)
    assert got.dtype == dtype and got.shape == (40, 1024)
    if dtype == torch.float32:
        assert torch.equal(got.cpu().view(torch.int32), want.view(torch.int32))
    else:
        assert torch.equal(got.cpu().view(torch.int16), want.to(dtype).view(torch.int16))


def test_dequantize_default_dtype_and_bf16_storage(ops):
    vals = torch.tensor([0.0, -0.0, 1.5, -2.25, float("inf"), float("-inf"), 3.0e38, 1e-40] * 4, dtype=torch.float32)
    bf = vals.to(torch.bfloat16)
    raw = bf.view(torch.uint8).cuda()
    out = ops.dequantize(raw, 30, 2, 16, torch.float32)
    assert torch.equal(out.cpu().reshape(-1), bf.to(torch.float32))
    q = ops.quantize(torch.zeros((2, 256), device="cuda"), 12)
    assert ops.dequantize(q.reshape(-1), 12, 2, 256, None).dtype == torch.float16
    # odd length bf16 rows exercise the scalar tail
    out = ops.dequantize(bf[:21].view(torch.uint8).cuda(), 30, 3, 7, torch.float16)
    assert torch.equal(out.cpu().reshape(-1), bf[:21].to(torch.float16))


def test_quantize_on_a_side_stream_and_leading_dims(ops, checker):
    x = np.random.default_rng(2).standard_normal((2, 3, 512), dtype=np.float32)
    xt = torch.from_numpy(x).cuda()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        q = ops.quantize(xt, 12)
    s.synchronize()
    assert q.shape == (2, 3, 288) and q.dtype == torch.uint8
    np.testing.assert_array_equal(q.cpu().numpy(), checker.quantize_rows(x, 12))


def test_optional_imatrix_upstream_behaviour_and_the_weighted_op(ops, checker):
    """`quantize` is upstream's op: a type that can do without importance weights ignores them
    (upstream cuda_quantize.cu:37-49); `quantize_weighted` applies them like the CPU quantizer does."""
    x, im = inputs.lattice_matrix(8, 1024)
    xt, imt = torch.from_numpy(x).cuda(), torch.from_numpy(im).cuda()
    plain = checker.quantize_rows(x, 12)
    weighted = checker.quantize_rows(x, 12, im)
    assert not np.array_equal(plain, weighted)
    np.testing.assert_array_equal(ops.quantize(xt, 12, imt).cpu().numpy(), plain)
    np.testing.assert_array_equal(torch.ops._C_gguf.quantize(xt, 12, imt).cpu().numpy(), plain)
    np.testing.assert_array_equal(ops.quantize_weighted(xt, 12, imt).cpu().numpy(), weighted)
    # a type that needs the weights reads them through either entry point
    need = checker.quantize_rows(x, 16, im)
    np.testing.assert_array_equal(ops.quantize(xt, 16, imt).cpu().numpy(), need)
    np.testing.assert_array_equal(ops.quantize_weighted(xt, 16, imt).cpu().numpy(), need)


def test_argument_rejection(ops):
    w = torch.zeros((2, 256), device="cuda")
    with pytest.raises(RuntimeError, match="expects a CUDA tensor"):
        ops.quantize(torch.zeros((2, 256)), 12)
    with pytest.raises(RuntimeError, match="expects float32 input"):
        ops.quantize(w.half(), 12)
    with pytest.raises(RuntimeError, match="expects contiguous input"):
        ops.quantize(torch.zeros((256, 2), device="cuda").t(), 12)
    with pytest.raises(RuntimeError, match="Unsupported GGML quantization type for CUDA quantize: 15"):
        ops.quantize(w, 15)
    with pytest.raises(RuntimeError, match="Unsupported GGML quantization type for CUDA quantize: 99"):
        ops.quantize(w, 99)
    with pytest.raises(RuntimeError, match="must be divisible by the quantization block size"):
        ops.quantize(torch.zeros((2, 100), device="cuda"), 12)
    with pytest.raises(RuntimeError, match="requires imatrix for GGML quantization type: 16"):
        ops.quantize(w, 16)
    with pytest.raises(RuntimeError, match="imatrix must be a CUDA tensor"):
        ops.quantize(w, 16, torch.ones(256))
    with pytest.raises(RuntimeError, match="imatrix must be float32"):
        ops.quantize(w, 16, torch.ones(256, device="cuda", dtype=torch.float16))
    with pytest.raises(RuntimeError, match="imatrix must be one-dimensional"):
        ops.quantize(w, 16, torch.ones((1, 256), device="cuda"))
    with pytest.raises(RuntimeError, match="at least input width elements"):
        ops.quantize(w, 16, torch.ones(128, device="cuda"))
    q = torch.zeros(288, dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError, match="expects uint8 input"):
        ops.dequantize(q.float(), 12, 2, 256, None)
    with pytest.raises(RuntimeError, match="positive row count"):
        ops.dequantize(q, 12, 0, 256, None)
    with pytest.raises(RuntimeError, match="positive row width"):
        ops.dequantize(q, 12, 2, 0, None)
    with pytest.raises(RuntimeError, match="output dtype must be float16, bfloat16, or float32"):
        ops.dequantize(q, 12, 2, 256, torch.float64)
    with pytest.raises(RuntimeError, match="Unsupported GGML quantization type for CUDA dequantize: 15"):
        ops.dequantize(q, 15, 2, 256, None)
    with pytest.raises(RuntimeError, match="output width must be divisible"):
        ops.dequantize(q, 12, 2, 100, None)
    with pytest.raises(RuntimeError, match="input has 288 bytes, expected 432"):
        ops.dequantize(q, 12, 3, 256, None)


def test_native_context_buffers_events_and_rows(checker):
    """libgguf_cuda_* with a library context: pinned host -> device -> quantize -> decode -> host."""
    from libgguf_b200._native import lib
    x = np.random.default_rng(9).standard_normal((48, 512), dtype=np.float32)
    want = checker.quantize_rows(x, 14)
    ctx = ctypes.c_void_p()
    assert lib.libgguf_cuda_context_create(0, ctypes.byref(ctx)) == 0
    try:
        d_in, d_q, d_out = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
        assert lib.libgguf_cuda_buffer_create(ctx, x.nbytes, ctypes.byref(d_in)) == 0
        assert lib.libgguf_cuda_buffer_create(ctx, 16, ctypes.byref(d_q)) == 0
        assert lib.libgguf_cuda_buffer_resize_discard(ctx, d_q, want.nbytes) == 0
        assert lib.libgguf_cuda_buffer_size(d_q) == want.nbytes
        assert lib.libgguf_cuda_buffer_create(ctx, x.size * 2, ctypes.byref(d_out)) == 0
        h = ctypes.c_void_p()
        assert lib.libgguf_cuda_host_buffer_create(ctx, x.nbytes, ctypes.byref(h)) == 0
        ctypes.memmove(lib.libgguf_cuda_host_buffer_data(h), x.ctypes.data, x.nbytes)
        e0, e1 = ctypes.c_void_p(), ctypes.c_void_p()
        assert lib.libgguf_cuda_event_create(ctx, ctypes.byref(e0)) == 0
        assert lib.libgguf_cuda_event_create(ctx, ctypes.byref(e1)) == 0
        assert lib.libgguf_cuda_event_record(ctx, e0) == 0
        assert lib.libgguf_cuda_h2d(ctx, d_in, 0, lib.libgguf_cuda_host_buffer_data(h), x.nbytes) == 0
        assert lib.libgguf_cuda_quantize_f32_rows(ctx, lib.libgguf_cuda_buffer_data(d_in), None,
                                                  lib.libgguf_cuda_buffer_data(d_q), 14, 48, 512) == 0
        assert lib.libgguf_cuda_dequantize_rows(ctx, lib.libgguf_cuda_buffer_data(d_q), 14, 48, 512, 1,
                                                lib.libgguf_cuda_buffer_data(d_out)) == 0
        got_q = np.empty_like(want)
        got_h = np.empty((48, 512), np.float16)
        assert lib.libgguf_cuda_d2h(ctx, got_q.ctypes.data, d_q, 0, want.nbytes) == 0
        assert lib.libgguf_cuda_d2h(ctx, got_h.ctypes.data, d_out, 0, got_h.nbytes) == 0
        assert lib.libgguf_cuda_event_record(ctx, e1) == 0
        assert lib.libgguf_cuda_event_synchronize(ctx, e1) == 0
        ms = ctypes.c_float(-1)
        assert lib.libgguf_cuda_event_elapsed_ms(ctx, e0, e1, ctypes.byref(ms)) == 0 and ms.value >= 0
        np.testing.assert_array_equal(got_q, want)
        ref_h = checker.dequantize_rows(want, 14, 512).astype(np.float16)
        np.testing.assert_array_equal(got_h.view(np.uint16), ref_h.view(np.uint16))
        # error reporting
        assert lib.libgguf_cuda_quantize_f32_rows(ctx, lib.libgguf_cuda_buffer_data(d_in), None,
                                                  lib.libgguf_cuda_buffer_data(d_q), 14, 48, 100) == 1
        assert b"not divisible" in lib.libgguf_cuda_last_error(ctx)
        assert lib.libgguf_cuda_quantize_f32_rows(ctx, lib.libgguf_cuda_buffer_data(d_in), None,
                                                  lib.libgguf_cuda_buffer_data(d_q), 16, 2, 256) == 1
        assert b"requires an imatrix" in lib.libgguf_cuda_last_error(ctx)
        assert lib.libgguf_cuda_quantize_f32_rows(ctx, lib.libgguf_cuda_buffer_data(d_in), None,
                                                  lib.libgguf_cuda_buffer_data(d_q), 15, 2, 256) == 2
        assert lib.libgguf_cuda_dequantize_rows(ctx, lib.libgguf_cuda_buffer_data(d_q), 14, 48, 512, 7,
                                                lib.libgguf_cuda_buffer_data(d_out)) == 2
        assert lib.libgguf_cuda_h2d(ctx, d_q, 8, x.ctypes.data, want.nbytes) == 1
        for ev in (e0, e1):
            lib.libgguf_cuda_event_destroy(ctx, ev)
        lib.libgguf_cuda_host_buffer_destroy(ctx, h)
        for b in (d_in, d_q, d_out):
            lib.libgguf_cuda_buffer_destroy(ctx, b)
    finally:
        lib.libgguf_cuda_context_destroy(ctx)


def test_dequantize_rows_on_stream_with_torch_stream(checker):
    from libgguf_b200._native import lib
    x = np.random.default_rng(4).standard_normal((16, 256), dtype=np.float32)
    enc = checker.quantize_rows(x, 8)
    src = torch.from_numpy(enc).cuda()
    out = torch.empty((16, 256), device="cuda", dtype=torch.float32)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    assert lib.libgguf_cuda_dequantize_rows_on_stream(src.data_ptr(), 8, 16, 256, 0, out.data_ptr(), s.cuda_stream) == 0
    s.synchronize()
    np.testing.assert_array_equal(out.cpu().numpy().view(np.uint32), checker.dequantize_rows(enc, 8, 256).view(np.uint32))


def test_misaligned_device_pointers(checker):
    """Encoded input and decoded output that start at odd addresses take the byte-granular paths."""
    from libgguf_b200._native import lib
    x = np.random.default_rng(6).standard_normal((9, 512), dtype=np.float32)
    for qtype in (8, 12, 14, 39):
        enc = checker.quantize_rows(x, qtype)
        buf = torch.zeros(enc.size + 64, dtype=torch.uint8, device="cuda")
        buf[3:3 + enc.size] = torch.from_numpy(enc.reshape(-1)).cuda()
        out = torch.zeros(9 * 512 + 8, dtype=torch.float16, device="cuda")
        st = lib.libgguf_cuda_dequantize_rows_on_stream(buf.data_ptr() + 3, qtype, 9, 512, 1, out.data_ptr() + 2,
                                                        torch.cuda.current_stream().cuda_stream)
        assert st == 0
        torch.cuda.synchronize()
        want = torch.from_numpy(checker.dequantize_rows(enc, qtype, 512)).to(torch.float16).reshape(-1)
        assert torch.equal(out[1:1 + 9 * 512].cpu().view(torch.int16), want.view(torch.int16))
        # quantize into a misaligned destination
        dst = torch.full((enc.size + 64,), 0xCD, dtype=torch.uint8, device="cuda")
        xt = torch.from_numpy(x).cuda()
        st = lib.libgguf_cuda_quantize_f32_rows_on_stream(xt.data_ptr(), None, dst.data_ptr() + 5, qtype,
                                                          9, 512, torch.cuda.current_stream().cuda_stream)
        assert st == 0
        torch.cuda.synchronize()
        got = dst.cpu().numpy()
        np.testing.assert_array_equal(got[5:5 + enc.size], enc.reshape(-1))
        assert (got[:5] == 0xCD).all() and (got[5 + enc.size:] == 0xCD).all()
