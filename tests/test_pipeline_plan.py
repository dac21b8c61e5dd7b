"""Shard planning of the conversion pipeline (no GPU needed)."""
import pytest

from libgguf_b200.convert import llama3_8b_plan, plan_shards


def test_shards_cover_every_row_exactly_once():
    tensors = [(12, 1000, 4096), (14, 7, 256), (8, 33, 32), (12, 0, 256)]
    shards = plan_shards(tensors, chunk_bytes=1 << 20)
    for ti, (_, rows, n) in enumerate(tensors):
        mine = sorted((r0, r) for t, r0, r in shards if t == ti)
        pos = 0
        for r0, r in mine:
            assert r0 == pos and r > 0
            assert r * n * 4 <= (1 << 20) or r == 1
            pos += r
        assert pos == rows
    sizes = [r * tensors[t][2] for t, _, r in shards]
    assert sizes == sorted(sizes, reverse=True)  # largest first


def test_row_wider_than_chunk_goes_alone():
    shards = plan_shards([(12, 5, 1 << 20)], chunk_bytes=1 << 20)
    assert sorted(shards) == [(0, i, 1) for i in range(5)]


def test_bad_descriptor():
    with pytest.raises(ValueError):
        plan_shards([(12, 4, 100)])
    with pytest.raises(ValueError):
        plan_shards([(15, 4, 256)])


def test_llama_plan_totals():
    plan = llama3_8b_plan()
    assert len(plan) == 2 + 32 * 7
    elems = sum(t.rows * t.cols for t in plan)
    assert elems == 8_029_995_008
    q6 = sum(t.rows * t.cols for t in plan if t.qtype == 14)
    assert q6 == 1_531_969_536 - 0 * 1  # output + half of attn_v and ffn_down
    shards = plan_shards([(t.qtype, t.rows, t.cols) for t in plan])
    assert sum(r * plan[t].cols for t, _, r in shards) == elems


def test_sixteen_bit_sources_fit_twice_the_rows_per_shard():
    wide = plan_shards([(12, 1024, 4096)], chunk_bytes=1 << 20)
    narrow = plan_shards([(12, 1024, 4096)], chunk_bytes=1 << 20, source_dtypes=[2])
    assert max(r for _, _, r in wide) == 64 and max(r for _, _, r in narrow) == 128
    assert sum(r for _, _, r in narrow) == 1024
    with pytest.raises(ValueError):
        plan_shards([(12, 4, 256)], source_dtypes=[7])
