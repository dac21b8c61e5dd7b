"""The multi-GPU conversion pipeline against the single-call path (bytes must not depend on the number of
workers, the chunk size, pinned vs pageable memory, or a worker failing half way)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


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
        with pytest.raises(RuntimeError, match="requires an imatrix"):
            pipe.quantize([(16, x, None, np.zeros(4 * 66, np.uint8))])
