"""The benchmark workloads' own data against the checker (the upstream CPU REF build): the microscaling matrix,
the decode sweep for every block type and both 16-bit outputs, and the conversion set's tensors through the
multi-GPU pipeline.  Zero tolerance: encoded bytes, fp32 bit patterns, and for fp16 / bf16 the bit patterns of
the round-to-nearest-even conversion of the checker's fp32 decode.  At the workloads' full sizes, where the CPU
checker would take minutes, slices are compared with the checker and the whole result is tied to the slices by
size-independent properties (a row range encodes to the same bytes whatever call it is part of)."""
import numpy as np
import pytest

import inputs

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

DTYPE_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


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


def _decode_on_gpu(enc: np.ndarray, qtype: int, width: int, dtype) -> "torch.Tensor":
    """Through the device-pointer C ABI (libgguf_cuda_dequantize_rows_on_stream) on torch's current stream."""
    from libgguf_b200._native import lib
    rows = enc.shape[0]
    dev_in = torch.from_numpy(enc).cuda()
    out = torch.empty((rows, width), dtype=dtype, device="cuda")
    st = lib.libgguf_cuda_dequantize_rows_on_stream(dev_in.data_ptr(), qtype, rows, width, DTYPE_CODE[dtype], out.data_ptr(),
                                                    torch.cuda.current_stream().cuda_stream)
    assert st == 0, lib.libgguf_cuda_thread_last_error().decode()
    torch.cuda.synchronize()
    return out.cpu()


def _same_bits(got: "torch.Tensor", want: "torch.Tensor") -> bool:
    view = torch.int32 if got.dtype == torch.float32 else torch.int16
    return torch.equal(got.view(view), want.view(view))


# ------------------------------------------------------------------------------------------------
# MXFP4 / NVFP4 workload: 8192 x 8192 Laplace(0, 0.01), bf16-origin, 1% of the blocks with a +-50 sigma outlier
@pytest.fixture(scope="module")
def microscaling():
    return inputs.microscaling_matrix()


@pytest.mark.parametrize("name", ["MXFP4", "NVFP4"])
def test_microscaling_workload(gguf, ops, checker, microscaling, name):
    """upstream csrc/quant/mxfp4.cpp:17-54, nvfp4.cpp:16-55 (encode), csrc/dequant/dequant.cpp:136-179 (decode)."""
    qtype = inputs.QTYPES[name]
    x = microscaling
    sigma50 = np.float32(50 * 0.01 * np.sqrt(2.0))
    # two 256-row slices; both hold outlier blocks (about 655 of their 65536 blocks each)
    slices = [slice(0, 256), slice(5000, 5256)]
    for sl in slices:
        assert (np.abs(x[sl]) >= sigma50 * np.float32(0.99)).sum() > 100
    whole = ops.quantize(torch.from_numpy(x).cuda(), qtype).cpu().numpy()            # the launch the benchmark times
    for sl in slices:
        want = checker.quantize_rows(x[sl], qtype)
        bad = np.flatnonzero((whole[sl] != want).any(axis=-1))
        assert bad.size == 0, f"{name}: {bad.size} rows of {sl} differ from the checker, first {bad[:5]}"
        np.testing.assert_array_equal(gguf.quantize_rows(x[sl], qtype), want)            # host-pointer ABI
        ref32 = torch.from_numpy(checker.dequantize_rows(want, qtype, x.shape[1]))
        assert _same_bits(_decode_on_gpu(want, qtype, x.shape[1], torch.float32), ref32)
        assert _same_bits(_decode_on_gpu(want, qtype, x.shape[1], torch.bfloat16), ref32.to(torch.bfloat16))
    # the whole matrix: a row range quantized alone gives the bytes it has inside the full call
    np.testing.assert_array_equal(ops.quantize(torch.from_numpy(x[3000:3100]).cuda(), qtype).cpu().numpy(), whole[3000:3100])
    # and the full-size bf16 decode equals the slice-wise decode on the rows the checker saw
    full_bf16 = _decode_on_gpu(whole, qtype, x.shape[1], torch.bfloat16)
    want = checker.quantize_rows(x[slices[1]], qtype)
    ref = torch.from_numpy(checker.dequantize_rows(want, qtype, x.shape[1])).to(torch.bfloat16)
    assert _same_bits(full_bf16[slices[1]], ref)


# ------------------------------------------------------------------------------------------------
# decode sweep: N(0, 0.02) rows at width 4096, encoded by the checker, decoded to fp16 and bf16 on the GPU
@pytest.fixture(scope="module")
def sweep_rows():
    return inputs.decode_sweep_matrix(512)


@pytest.mark.parametrize("name", sorted(inputs.QTYPES))
def test_decode_sweep_rows_every_type_to_fp16_and_bf16(checker, sweep_rows, name):
    qtype = inputs.QTYPES[name]
    lattice = name.startswith(("IQ1", "IQ2", "IQ3"))
    x = sweep_rows[:96] if lattice else sweep_rows    # the CPU lattice encoders take seconds per hundred rows
    im = inputs.imatrix_for(4096, seed=3) if checker.requires_imatrix(qtype) else None
    enc = checker.quantize_rows(x, qtype, im)
    ref32 = torch.from_numpy(checker.dequantize_rows(enc, qtype, 4096))
    for dtype in (torch.float16, torch.bfloat16, torch.float32):
        got = _decode_on_gpu(enc, qtype, 4096, dtype)
        assert _same_bits(got, ref32.to(dtype)), (name, dtype)


@pytest.mark.parametrize("name", ["Q8_0", "Q4_K"])
def test_decode_sweep_at_full_height(checker, name):
    """All 14336 rows (the 7168-CTA grid of the benchmark) for two of the six types: every element against the
    checker's decode of the checker's bytes."""
    qtype = inputs.QTYPES[name]
    x = inputs.decode_sweep_matrix()
    enc = checker.quantize_rows(x, qtype)
    ref32 = torch.from_numpy(checker.dequantize_rows(enc, qtype, 4096))
    for dtype in (torch.float16, torch.bfloat16):
        assert _same_bits(_decode_on_gpu(enc, qtype, 4096, dtype), ref32.to(dtype)), (name, dtype)


# ------------------------------------------------------------------------------------------------
# conversion set: one tensor of each distinct shape with the x20 outlier columns through the pipeline, 2 workers
def test_conversion_tensors_through_the_pipeline_match_the_checker(gguf, checker):
    from libgguf_b200.convert import ConversionPipeline
    ndev = torch.cuda.device_count()
    q4, q6 = inputs.QTYPES["Q4_K"], inputs.QTYPES["Q6_K"]
    cases = [("blk.0.attn_k", 1024, 4096, None, q4), ("blk.0.attn_v", 1024, 4096, None, q6),
             ("blk.0.ffn_down", 4096, 14336, 384, q6), ("blk.1.ffn_down", 4096, 14336, 384, q4),
             ("blk.0.ffn_gate", 14336, 4096, 1536, q4), ("output", 128256, 4096, 1024, q6),
             ("token_embd", 128256, 4096, 1024, q4)]
    batch = []
    for name, rows, width, first, qtype in cases:
        x = inputs.conversion_tensor(name, rows, width, first)
        # the outlier channels are there: about 0.1% of the columns carry 20x the spread
        col_rms = np.sqrt((x.astype(np.float64) ** 2).mean(axis=0))
        assert (col_rms > 0.2).sum() == -(-width // 1000)
        dst = np.empty(x.shape[0] * gguf.row_size(qtype, width), np.uint8)
        batch.append((qtype, x, None, dst))
    with ConversionPipeline([0, 1 % ndev], slots=3, chunk_bytes=4 << 20) as pipe:
        pipe.quantize(batch)
        stats = pipe.stats()
    assert sum(stats["shards_per_device"]) > len(batch)      # tensors were cut into row-range shards
    for (name, *_), (qtype, x, _, dst) in zip(cases, batch):
        want = checker.quantize_rows(x, qtype)
        got = dst.reshape(want.shape)
        bad = np.flatnonzero((got != want).any(axis=-1))
        assert bad.size == 0, f"{name}: {bad.size} rows differ from the checker, first {bad[:5]}"
    # 16-bit sources (uploaded as 16-bit, widened on the GPU) against the checker fed the host-widened copy
    x = inputs.conversion_tensor("blk.2.attn_q", 4096, 4096, 512)
    bf = (x.view(np.uint32) >> np.uint32(16)).astype(np.uint16)
    widened = (bf.astype(np.uint32) << np.uint32(16)).view(np.float32)
    dst = np.empty(512 * gguf.row_size(q4, 4096), np.uint8)
    with ConversionPipeline([0, 1 % ndev], slots=3, chunk_bytes=1 << 20) as pipe:
        pipe.quantize([(q4, bf, None, dst)])
    np.testing.assert_array_equal(dst.reshape(512, -1), checker.quantize_rows(widened, q4))


# ------------------------------------------------------------------------------------------------
# block scales at the edges of fp16, every type, all three output types
_D_OFFSET = {"Q4_0": 0, "Q4_1": 0, "Q5_0": 0, "Q5_1": 0, "Q8_0": 0, "Q1_0": 0, "Q2_K": 80, "Q3_K": 108, "Q4_K": 0, "Q5_K": 0,
             "Q6_K": 208, "TQ1_0": 52, "TQ2_0": 64, "IQ2_XXS": 0, "IQ2_XS": 0, "IQ2_S": 0, "IQ3_XXS": 0, "IQ3_S": 0, "IQ1_S": 0,
             "IQ4_NL": 0, "IQ4_XS": 0}
_BLOCK_BYTES = {"Q4_0": 18, "Q4_1": 20, "Q5_0": 22, "Q5_1": 24, "Q8_0": 34, "Q1_0": 18, "Q2_K": 84, "Q3_K": 110, "Q4_K": 144,
                "Q5_K": 176, "Q6_K": 210, "TQ1_0": 54, "TQ2_0": 66, "IQ2_XXS": 66, "IQ2_XS": 74, "IQ2_S": 82, "IQ3_XXS": 98,
                "IQ3_S": 110, "IQ1_S": 50, "IQ4_NL": 18, "IQ4_XS": 136}


@pytest.mark.parametrize("name", sorted(_D_OFFSET))
def test_decode_with_block_scales_at_the_edges_of_fp16(checker, name):
    """Valid encodings whose fp16 block scale is overwritten with zero, minus zero, the smallest and largest subnormal,
    the smallest normal, 65504, infinity and negative values: the 16-bit decoders that select precomputed patterns
    (and the arithmetic ones) must still give the correctly rounded fp32 decode; where the fp32 value is NaN
    (infinity times zero) the output must be NaN too."""
    qtype = inputs.QTYPES[name]
    width = 2048
    x = np.random.default_rng(41).standard_normal((16, width), dtype=np.float32)
    im = inputs.imatrix_for(width, seed=5) if checker.requires_imatrix(qtype) else None
    enc = checker.quantize_rows(x, qtype, im).copy()
    scales = np.array([0x0000, 0x8000, 0x0001, 0x03FF, 0x0400, 0x7BFF, 0x7C00, 0xFC00, 0xBC00, 0x8001, 0x3C00, 0xFBFF], np.uint16)
    blocks = enc.reshape(-1, _BLOCK_BYTES[name])
    pick = np.arange(blocks.shape[0]) % (len(scales) + 3)      # some blocks keep their own scale
    for i, s in enumerate(scales):
        rows = pick == i
        blocks[rows, _D_OFFSET[name]] = s & 0xFF
        blocks[rows, _D_OFFSET[name] + 1] = s >> 8
    with np.errstate(all="ignore"):
        ref32 = torch.from_numpy(checker.dequantize_rows(enc, qtype, width))
    for dtype in (torch.float32, torch.float16, torch.bfloat16):
        got = _decode_on_gpu(enc, qtype, width, dtype)
        want = ref32.to(dtype)
        nan = torch.isnan(want)
        assert torch.equal(torch.isnan(got), nan), (name, dtype)
        view = torch.int32 if dtype == torch.float32 else torch.int16
        assert torch.equal(got.view(view)[~nan], want.view(view)[~nan]), (name, dtype)
