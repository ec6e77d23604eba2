"""Host logic of the host-buffer pipeline: chunk dimension and ranges (no GPU needed)."""
from flashbias_b200.host_pipeline import plan_chunks

MB = 1 << 20


def _covers(ranges, n):
    return ranges[0][0] == 0 and ranges[-1][1] == n and all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))


def test_heads_when_factors_are_per_head():
    dim, ranges = plan_chunks((1, 8192, 50, 32), (1, 8192, 50, 2), (1, 8192, 50, 2), 108 * MB, 5)
    assert dim == "head" and len(ranges) == 5 and _covers(ranges, 50)
    assert max(hi - lo for lo, hi in ranges) - min(hi - lo for lo, hi in ranges) <= 1


def test_batch_when_factors_are_shared_over_heads():
    dim, ranges = plan_chunks((2, 32768, 8, 64), (2, 32768, 1, 5), (2, 32768, 1, 5), 270 * MB, 5)
    assert dim == "batch" and ranges == [(0, 1), (1, 2)]


def test_single_chunk_when_no_dimension_is_free_or_the_problem_is_small():
    assert plan_chunks((1, 4096, 8, 32), (1, 4096, 1, 4), (1, 4096, 1, 4), 64 * MB, 5) == ("none", [(0, 1)])
    assert plan_chunks((2, 1024, 4, 32), (2, 1024, 4, 8), (2, 1024, 4, 8), 2 * MB, 5) == ("none", [(0, 4)])


def test_no_factors_and_chunk_count_capped_by_bytes():
    dim, ranges = plan_chunks((4, 2048, 16, 64), None, None, 13 * MB, 5)
    assert dim == "head" and len(ranges) == 3 and _covers(ranges, 16)


def test_head_chunks_keep_rows_of_at_least_512_bytes():
    # 6 heads of head_dim 64 are 768-byte rows: cutting them would leave 256-byte rows for the 2-D copies
    assert plan_chunks((4, 2048, 6, 64), None, None, 13 * MB, 5) == ("none", [(0, 6)])
    # a rank's slab of the ALiBi problem on 8 GPUs: 7 heads of head_dim 32 = 448-byte rows -> one chunk
    assert plan_chunks((1, 8192, 7, 32), (1, 8192, 7, 2), (1, 8192, 7, 2), 15 * MB, 5) == ("none", [(0, 7)])
    # the whole problem on one GPU: 50 heads -> 5 chunks of 10 heads (640-byte rows)
    assert len(plan_chunks((1, 8192, 50, 32), (1, 8192, 50, 2), (1, 8192, 50, 2), 108 * MB, 5)[1]) == 5
