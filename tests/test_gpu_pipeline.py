"""The multi-GPU conversion pipeline against the single-call path (bytes must not depend on the number of
workers, the chunk size, pinned vs pageable memory, or a worker failing half way)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def checker():
    from oracle import reference
    if reference.available("ref"):
        return reference.load("ref")
    import subprocess
    from pathlib import Path
    if not reference.available("port"):
        subprocess.run(["make", "-C", str(Path(__file__).parents[1] / "oracle"), "oracle"], check=True, capture_output=True)
    return reference.load("port")


def _tensors(rng, pinned):
    specs = [(12, 300, 1024), (14, 130, 512), (8, 77, 256), (10, 64, 768), (18, 40, 512)]
    out = []
    for qtype, rows, n in specs:
        x = rng.standard_normal((rows, n), dtype=np.float32)
        if pinned:
            t = torch.from_numpy(x).pin_memory()
            x = t.numpy()
            out.append((qtype, x, t))
        else:
            out.append((qtype, x, None))
    return out


@pytest.mark.parametrize("pinned", [False, True])
@pytest.mark.parametrize("workers", [1, 2, 3])
def test_pipeline_matches_single_calls(gguf, pinned, workers):
    from libgguf_b200.convert import ConversionPipeline
    rng = np.random.default_rng(1)
    ndev = torch.cuda.device_count()
    devices = [i % ndev for i in range(workers)]
    items = _tensors(rng, pinned)
    im = (rng.chisquare(4, 512) / 4).astype(np.float32)
    batch, keep = [], []
    for qtype, x, holder in items:
        rs = gguf.row_size(qtype, x.shape[1])
        if pinned:
            d = torch.empty(x.shape[0] * rs, dtype=torch.uint8).pin_memory()
            keep.append(d)
            dst = d.numpy()
        else:
            dst = np.empty(x.shape[0] * rs, np.uint8)
        batch.append((qtype, x, im if qtype == 18 else None, dst))
    with ConversionPipeline(devices, slots=2, chunk_bytes=64 << 10) as pipe:
        pipe.quantize(batch)
        stats = pipe.stats()
    assert sum(stats["shards_per_device"]) > len(batch)
    for qtype, x, imx, dst in batch:
        want = gguf.quantize_rows(x, qtype, imx)
        np.testing.assert_array_equal(dst.reshape(want.shape), want)


def test_failed_worker_hands_its_shards_to_the_others(gguf):
    from libgguf_b200.convert import ConversionPipeline
    rng = np.random.default_rng(2)
    ndev = torch.cuda.device_count()
    x = rng.standard_normal((512, 1024), dtype=np.float32)
    dst = np.zeros(512 * gguf.row_size(12, 1024), np.uint8)
    with ConversionPipeline([0, (1 % ndev)], slots=2, chunk_bytes=64 << 10) as pipe:
        pipe.inject_failure(0, 3)  # host-side: worker 0 reports an error after three shards
        pipe.quantize([(12, x, None, dst)])
        stats = pipe.stats()
    assert stats["requeued"] >= 1
    np.testing.assert_array_equal(dst.reshape(512, -1), gguf.quantize_rows(x, 12))
    # every worker failing is an error, not a hang
    with ConversionPipeline([0], slots=2, chunk_bytes=64 << 10) as pipe:
        pipe.inject_failure(0, 1)
        with pytest.raises(RuntimeError, match="injected failure"):
            pipe.quantize([(12, x, None, dst)])


def test_pipeline_rejects_bad_batches(gguf):
    from libgguf_b200.convert import ConversionPipeline
    x = np.zeros((4, 256), np.float32)
    with ConversionPipeline([0]) as pipe:
        with pytest.raises(ValueError):
            pipe.quantize([(12, x, None, np.zeros(10, np.uint8))])


@pytest.mark.parametrize("kind", ["float32", "float16"])
def test_missing_importance_weights_are_derived_from_the_tensor(gguf, checker, kind):
    """A type that requires an imatrix and gets none: the pipeline takes the column sums of squares of the whole
    tensor (row order, like upstream) and quantizes with them, whatever the shard size."""
    from libgguf_b200.convert import ConversionPipeline
    rng = np.random.default_rng(9)
    x = (rng.standard_normal((150, 512)) * 0.3).astype(np.float32)
    src = x.astype(np.float16) if kind == "float16" else x
    wide = src.astype(np.float32)
    weights = np.sum(wide * wide, axis=0, dtype=np.float32)
    assert np.array_equal(gguf.auto_imatrix(wide).view(np.uint32), weights.view(np.uint32))
    for qtype in (16, 19):
        dst = np.zeros(150 * gguf.row_size(qtype, 512), np.uint8)
        # two workers, on two GPUs where the box has them: per-device kernel settings must hold on every device
        with ConversionPipeline([0, 1 % torch.cuda.device_count()], slots=2, chunk_bytes=40 << 10) as pipe:
            pipe.quantize([(qtype, src, None, dst)])
        want = checker.quantize_rows(wide, qtype, weights)
        assert np.array_equal(dst, np.ascontiguousarray(want).view(np.uint8).reshape(-1))
        assert np.array_equal(gguf.quantize_rows(wide, qtype).reshape(-1), dst)


def test_accumulate_imatrix_entry_point_continues_a_running_sum(gguf):
    from libgguf_b200._native import lib
    rng = np.random.default_rng(10)
    x = rng.standard_normal((333, 200)).astype(np.float32)
    want = np.sum(x * x, axis=0, dtype=np.float32)
    d = torch.from_numpy(x).cuda()
    acc = torch.zeros(200, dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    for r0, r1 in ((0, 100), (100, 101), (101, 333)):
        assert lib.libgguf_cuda_accumulate_imatrix_on_stream(d[r0:r1].data_ptr(), r1 - r0, 200, acc.data_ptr(), stream) == 0
    assert np.array_equal(acc.cpu().numpy().view(np.uint32), want.view(np.uint32))
    assert lib.libgguf_cuda_accumulate_imatrix_on_stream(d.data_ptr(), 1, 0, acc.data_ptr(), stream) != 0


@pytest.mark.parametrize("kind", ["float16", "bfloat16"])
def test_sixteen_bit_sources_are_widened_on_the_gpu(gguf, kind):
    """fp16 / bf16 source rows go through the pipeline as 16-bit values; the bytes must equal quantizing the
    host-widened fp32 copy (what upstream's converter uploads)."""
    from libgguf_b200.convert import ConversionPipeline
    rng = np.random.default_rng(5)
    batch, want = [], []
    for qtype, rows, n in [(12, 300, 1024), (8, 77, 256), (14, 130, 512), (39, 33, 64), (2, 5, 32)]:
        x = rng.standard_normal((rows, n), dtype=np.float32)
        x[0, :4] = [0.0, -0.0, 65504.0, 6e-8]
        if kind == "float16":
            src = x.astype(np.float16)
            wide = src.astype(np.float32)
        else:
            src = (x.view(np.uint32) >> 16).astype(np.uint16)  # truncated bf16 bit patterns
            wide = (src.astype(np.uint32) << 16).view(np.float32)
        dst = np.zeros(rows * gguf.row_size(qtype, n), dtype=np.uint8)
        batch.append((qtype, np.ascontiguousarray(src), None, dst))
        want.append(gguf.quantize_rows(wide, qtype).reshape(-1))
    with ConversionPipeline([0], slots=2, chunk_bytes=64 << 10) as pipe:
        pipe.quantize(batch)
    for (_, _, _, dst), w in zip(batch, want):
        assert np.array_equal(dst, w.view(np.uint8).reshape(-1))


def test_widen_and_quantize_from_entry_points(gguf):
    import ctypes
    from libgguf_b200._native import lib
    rng = np.random.default_rng(6)
    x = rng.standard_normal((64, 512), dtype=np.float32)
    half = torch.from_numpy(x.astype(np.float16)).cuda()
    bf = torch.from_numpy(x).cuda().to(torch.bfloat16)
    stream = torch.cuda.current_stream().cuda_stream
    for code, t in ((1, half), (2, bf)):
        wide = torch.empty(t.shape, dtype=torch.float32, device="cuda")
        assert lib.libgguf_cuda_widen_on_stream(t.data_ptr(), code, wide.data_ptr(), t.numel(), stream) == 0
        assert torch.equal(wide, t.float())
        # one element past a 16-byte boundary: the scalar path
        assert lib.libgguf_cuda_widen_on_stream(t.data_ptr() + 2, code, wide.data_ptr() + 4, t.numel() - 1, stream) == 0
        assert torch.equal(wide.reshape(-1)[1:], t.float().reshape(-1)[1:])
        out = torch.empty(64 * gguf.row_size(12, 512), dtype=torch.uint8, device="cuda")
        scratch = torch.empty(t.shape, dtype=torch.float32, device="cuda")
        assert lib.libgguf_cuda_quantize_rows_from_on_stream(t.data_ptr(), code, scratch.data_ptr(), None, out.data_ptr(), 12, 64, 512, stream) == 0
        want = gguf.quantize_rows(t.float().cpu().numpy(), 12)
        assert np.array_equal(out.cpu().numpy(), want.reshape(-1))
    assert lib.libgguf_cuda_widen_on_stream(half.data_ptr(), 0, wide.data_ptr(), 8, stream) != 0
    assert lib.libgguf_cuda_quantize_rows_from_on_stream(half.data_ptr(), 1, None, None, out.data_ptr(), 12, 64, 512, stream) != 0
