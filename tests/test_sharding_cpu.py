"""Host logic of the multi-GPU partition, exercised with two gloo ranks on the CPU (the attention
callable is the CPU checker here; on GPU ranks it is flash_bias_func)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flashbias_b200.sharding import bh_segments, shard_query_blocks, shard_ranges, sharded_attention, gather_bh
from oracle import flashbias_oracle as orc


def test_shard_ranges_cover_exactly_once():
    for n, w in [(50, 8), (8, 8), (16, 8), (5, 8), (98304, 8), (7, 2)]:
        r = shard_ranges(n, w)
        assert r[0][0] == 0 and r[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(r, r[1:]))
        sizes = [b - a for a, b in r]
        assert max(sizes) - min(sizes) <= 1
    assert [b - a for a, b in shard_ranges(50, 8)] == [7, 7, 6, 6, 6, 6, 6, 6]


def test_bh_segments_partition_batch_heads():
    B, H, world = 3, 5, 4
    seen = set()
    for r in range(world):
        for (b, h0, h1) in bh_segments(B, H, r, world):
            for h in range(h0, h1):
                assert (b, h) not in seen
                seen.add((b, h))
    assert seen == {(b, h) for b in range(B) for h in range(H)}


def test_query_blocks_round_robin():
    blocks = [shard_query_blocks(1536, r, 8) for r in range(8)]
    flat = sorted(x for b in blocks for x in b)
    assert flat[0][0] == 0 and flat[-1][1] == 1536 and len(flat) == 12
    assert all(a[1] == b[0] for a, b in zip(flat, flat[1:]))


def _oracle_fn(q, k, v, qb, kb, mask, causal, scale):
    return orc.attention_forward(q, k, v, qb, kb, mask, causal, scale)[0]


def _worker(rank, world, port, q, k, v, qb, kb, want):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        pieces = sharded_attention(_oracle_fn, q, k, v, qb, kb, None, True, 0.3, rank=rank, world=world)
        full = gather_bh(pieces, *q.shape)
        # shards are independent problems: the assembled result equals the unsharded one bit for bit
        assert torch.equal(full, want)
        # barrier + max-reduce, as the benchmark does for its timings
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert t.item() == world
    finally:
        dist.destroy_process_group()


def test_two_rank_sharded_equals_single(tmp_path):
    g = torch.Generator().manual_seed(3)
    B, S, H, D, R = 2, 40, 3, 16, 4
    q, k, v = (torch.randn(B, S, H, D, generator=g) for _ in range(3))
    qb = torch.randn(1, S, H, R, generator=g)      # batch-broadcast factor
    kb = torch.randn(B, S, 1, R, generator=g)      # head-broadcast factor
    want = _oracle_fn(q, k, v, qb, kb, None, True, 0.3)
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, q, k, v, qb, kb, want), nprocs=2, join=True)
