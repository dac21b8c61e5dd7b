"""`torch.ops._C_gguf.quantize / dequantize` on the meta device and under FakeTensorMode: shapes, dtypes, devices
and the argument checks, without a GPU.  The cases are those of upstream
tests/backends/libgguf_cuda/test_cuda_fake_ops.py (meta shapes :101-126, quantize validation :129-279, dequantize
:282-424), driven through this repository's registration of the same operator names and schemas
(upstream src/libgguf/libgguf_cuda/csrc/torch_bindings.cpp:12-20)."""
from contextlib import nullcontext

import pytest

torch = pytest.importorskip("torch")
from torch._subclasses.fake_tensor import FakeTensorMode  # noqa: E402

import libgguf_b200 as libgguf  # noqa: E402
from libgguf_b200 import GGML_QUANT_SIZES, GGMLQuantizationType as T  # noqa: E402
from libgguf_b200 import libgguf_cuda  # noqa: E402

QUANT = [T.IQ2_XXS, T.IQ2_XS, T.IQ2_S, T.IQ3_XXS, T.IQ3_S, T.IQ1_S, T.IQ1_M, T.IQ4_NL, T.IQ4_XS, T.MXFP4, T.NVFP4, T.Q1_0,
         T.Q2_K, T.Q3_K, T.Q4_0, T.Q4_1, T.Q4_K, T.Q5_0, T.Q5_1, T.Q5_K, T.Q6_K, T.Q8_0, T.TQ1_0, T.TQ2_0]
NEED_IMATRIX = [q for q in QUANT if libgguf.quantize_requires_imatrix(q)]
DEQUANT = QUANT + [T.BF16]
MODES = ("meta", "fake")


def ctx(mode):
    return (nullcontext(), "meta") if mode == "meta" else (FakeTensorMode(), "cuda")


def test_operators_are_registered_with_upstreams_schemas():
    assert str(torch.ops._C_gguf.quantize.default._schema) == "_C_gguf::quantize(Tensor W, int type, Tensor? imatrix=None) -> Tensor"
    assert str(torch.ops._C_gguf.dequantize.default._schema) == \
        "_C_gguf::dequantize(Tensor W, int type, SymInt m, SymInt n, ScalarType? dtype) -> Tensor"
    assert NEED_IMATRIX == [T.IQ2_XXS, T.IQ2_XS, T.IQ1_S]


@pytest.mark.parametrize("qtype", QUANT, ids=lambda q: q.name)
def test_quantize_meta_shape(qtype):
    block, size = GGML_QUANT_SIZES[qtype]
    width = block * 3
    rows = torch.empty((2, 3, width), device="meta", dtype=torch.float32)
    im = torch.empty((width,), device="meta", dtype=torch.float32) if qtype in NEED_IMATRIX else None
    out = libgguf_cuda.quantize(rows, int(qtype), im)
    assert out.device.type == "meta" and out.dtype == torch.uint8 and tuple(out.shape) == (2, 3, width * size // block)
    out = torch.ops._C_gguf.quantize(rows, int(qtype), im)
    assert tuple(out.shape) == (2, 3, width * size // block)


def test_quantize_fake_keeps_cuda_device():
    block, size = GGML_QUANT_SIZES[T.Q4_0]
    with FakeTensorMode():
        out = libgguf_cuda.quantize(torch.empty((4, block * 2), device="cuda", dtype=torch.float32), int(T.Q4_0))
    assert out.device.type == "cuda" and out.dtype == torch.uint8 and tuple(out.shape) == (4, 2 * size)


@pytest.mark.parametrize("mode", MODES)
def test_quantize_rejections(mode):
    context, device = ctx(mode)
    with context:
        f32 = dict(device=device, dtype=torch.float32)
        with pytest.raises(RuntimeError, match="at least one dimension"):
            libgguf_cuda.quantize(torch.empty((), **f32), int(T.Q4_0))
        with pytest.raises(RuntimeError, match="float32 input"):
            libgguf_cuda.quantize(torch.empty((1, 32), device=device, dtype=torch.float16), int(T.Q4_0))
        with pytest.raises(RuntimeError, match="divisible"):
            libgguf_cuda.quantize(torch.empty((1, 33), **f32), int(T.Q4_0))
        with pytest.raises(RuntimeError, match="Unsupported GGML quantization type"):
            libgguf_cuda.quantize(torch.empty((1, 32), **f32), int(T.F32))
        for qtype in NEED_IMATRIX:
            with pytest.raises(RuntimeError, match="requires imatrix"):
                libgguf_cuda.quantize(torch.empty((1, 256), **f32), int(qtype))
        q = int(NEED_IMATRIX[0])
        rows = torch.empty((1, 256), **f32)
        with pytest.raises(RuntimeError, match="imatrix must be a CUDA tensor"):
            libgguf_cuda.quantize(rows, q, torch.empty((256,), device="cpu", dtype=torch.float32))
        with pytest.raises(RuntimeError, match="imatrix must be float32"):
            libgguf_cuda.quantize(rows, q, torch.empty((256,), device=device, dtype=torch.float16))
        with pytest.raises(RuntimeError, match="one-dimensional"):
            libgguf_cuda.quantize(rows, q, torch.empty((1, 256), **f32))
        with pytest.raises(RuntimeError, match="at least input width elements"):
            libgguf_cuda.quantize(torch.empty((1, 512), **f32), q, torch.empty((256,), **f32))
        strided = torch.empty((256, 2), **f32)[:, 0]
        assert not strided.is_contiguous()
        with pytest.raises(RuntimeError, match="imatrix must be contiguous"):
            libgguf_cuda.quantize(rows, q, strided)


def test_quantize_fake_rejects_imatrix_on_another_device():
    with FakeTensorMode():
        rows = torch.empty((1, 256), device="cuda", dtype=torch.float32)
        with pytest.raises(RuntimeError, match="same device as input"):
            libgguf_cuda.quantize(rows, int(NEED_IMATRIX[0]), torch.empty((256,), device="meta", dtype=torch.float32))


@pytest.mark.parametrize("qtype", NEED_IMATRIX, ids=lambda q: q.name)
def test_quantize_fake_accepts_required_imatrix(qtype):
    block, size = GGML_QUANT_SIZES[qtype]
    with FakeTensorMode():
        out = libgguf_cuda.quantize(torch.empty((3, block * 2), device="cuda", dtype=torch.float32), int(qtype),
                                    torch.empty((block * 2,), device="cuda", dtype=torch.float32))
    assert out.device.type == "cuda" and tuple(out.shape) == (3, 2 * size)


def test_optional_imatrix_is_not_validated_by_quantize_but_is_by_quantize_weighted():
    """upstream's op looks at the weights only for the types that need them (cuda_quantize.cu:37-49)."""
    rows = torch.empty((2, 256), device="meta", dtype=torch.float32)
    bad = torch.empty((3,), device="meta", dtype=torch.float16)
    assert tuple(libgguf_cuda.quantize(rows, int(T.Q4_K), bad).shape) == (2, 144)
    with pytest.raises(RuntimeError, match="imatrix must be float32"):
        libgguf_cuda.quantize_weighted(rows, int(T.Q4_K), bad)
    good = torch.empty((256,), device="meta", dtype=torch.float32)
    assert tuple(libgguf_cuda.quantize_weighted(rows, int(T.Q4_K), good).shape) == (2, 144)


@pytest.mark.parametrize("qtype", DEQUANT, ids=lambda q: q.name)
@pytest.mark.parametrize("dtype", (None, torch.float32, torch.float16, torch.bfloat16))
def test_dequantize_meta(qtype, dtype):
    block, size = GGML_QUANT_SIZES[qtype]
    enc = torch.empty((5, size * 2), device="meta", dtype=torch.uint8)
    out = libgguf_cuda.dequantize(enc, int(qtype), 5, block * 2, dtype)
    assert out.device.type == "meta" and out.dtype == (dtype or torch.float16) and tuple(out.shape) == (5, block * 2)


def test_dequantize_fake_dtype_and_device():
    _, size = GGML_QUANT_SIZES[T.Q4_0]
    with FakeTensorMode():
        enc = torch.empty((2, size), device="cuda", dtype=torch.uint8)
        a = libgguf_cuda.dequantize(enc, int(T.Q4_0), 2, 32, None)
        b = libgguf_cuda.dequantize(enc, int(T.Q4_0), 2, 32, torch.float32)
        with pytest.raises(RuntimeError, match="expects a CUDA tensor"):
            libgguf_cuda.dequantize(torch.empty((2, size), device="cpu", dtype=torch.uint8), int(T.Q4_0), 2, 32, None)
    assert a.device.type == "cuda" and a.dtype == torch.float16 and tuple(a.shape) == (2, 32)
    assert b.dtype == torch.float32


@pytest.mark.parametrize("mode", MODES)
def test_dequantize_rejections(mode):
    context, device = ctx(mode)
    block, size = GGML_QUANT_SIZES[T.Q4_0]
    with context:
        enc = torch.empty((2, size), device=device, dtype=torch.uint8)
        with pytest.raises(RuntimeError, match="uint8 input"):
            libgguf_cuda.dequantize(torch.empty((2, size), device=device, dtype=torch.float32), int(T.Q4_0), 2, 32, None)
        with pytest.raises(RuntimeError, match="float16, bfloat16, or float32"):
            libgguf_cuda.dequantize(enc, int(T.Q4_0), 2, 32, torch.int32)
        with pytest.raises(RuntimeError, match="Unsupported GGML quantization type"):
            libgguf_cuda.dequantize(torch.empty((2, 128), device=device, dtype=torch.uint8), int(T.F32), 2, 32, None)
        with pytest.raises(RuntimeError, match="positive row count"):
            libgguf_cuda.dequantize(enc, int(T.Q4_0), 0, 32, None)
        with pytest.raises(RuntimeError, match="positive row width"):
            libgguf_cuda.dequantize(enc, int(T.Q4_0), 2, 0, None)
        with pytest.raises(RuntimeError, match="divisible"):
            libgguf_cuda.dequantize(enc, int(T.Q4_0), 2, block + 1, None)
        with pytest.raises(RuntimeError, match=r"input has .* bytes, expected"):
            libgguf_cuda.dequantize(torch.empty((2, size + 1), device=device, dtype=torch.uint8), int(T.Q4_0), 2, 32, None)
        with pytest.raises(RuntimeError, match=r"input has .* bytes, expected"):
            libgguf_cuda.dequantize(torch.empty((), device=device, dtype=torch.uint8), int(T.BF16), 1, 1, None)


def test_cpu_tensors_are_refused_in_upstreams_words():
    with pytest.raises(RuntimeError, match="CUDA quantize expects a CUDA tensor"):
        libgguf_cuda.quantize(torch.zeros((2, 256)), int(T.Q4_K))
    with pytest.raises(RuntimeError, match="CUDA dequantize expects a CUDA tensor"):
        libgguf_cuda.dequantize(torch.zeros(288, dtype=torch.uint8), int(T.Q4_K), 2, 256, None)


def test_export_traces_through_the_operator():
    """A module that decodes a stored weight can be traced with fake tensors: the graph holds the operator."""
    from torch.fx.experimental.proxy_tensor import make_fx

    def f(enc):
        return libgguf_cuda.dequantize(enc, int(T.Q4_K), 4, 256, torch.bfloat16) * 2

    with FakeTensorMode() as mode:
        enc = torch.empty((4 * 144,), device="cuda", dtype=torch.uint8)
    graph = make_fx(f, tracing_mode="fake")(enc)
    assert "_C_gguf.dequantize" in graph.code
