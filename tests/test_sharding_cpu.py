"""Host logic of the multi-GPU partition, exercised with two gloo ranks on the CPU (the attention
callable is the CPU checker here; on GPU ranks it is flash_bias_func)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flashbias_b200.sharding import (allreduce_shared_factor_grads, bh_segments, gather_bh, shard_query_blocks,
                                     shard_ranges, shared_factor_flags, sharded_attention,
                                     sharded_forward_backward)
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


def test_bh_slabs_merge_whole_batch_entries():
    from flashbias_b200.sharding import bh_slabs
    assert bh_slabs(4096, 24, 3, 8) == [(1536, 2048, 0, 24)]           # swin: 512 whole batch entries
    assert bh_slabs(1, 50, 0, 8) == [(0, 1, 0, 7)] and bh_slabs(1, 50, 7, 8) == [(0, 1, 44, 50)]
    assert bh_slabs(2, 8, 5, 8) == [(1, 2, 2, 4)]                        # pde: 2 heads of batch entry 1
    seen = set()
    for r in range(4):                                                   # mixed: 3 batch entries x 5 heads over 4
        for (b0, b1, h0, h1) in bh_slabs(3, 5, r, 4):
            for b in range(b0, b1):
                for h in range(h0, h1):
                    assert (b, h) not in seen
                    seen.add((b, h))
    assert len(seen) == 15


def test_query_blocks_round_robin():
    blocks = [shard_query_blocks(1536, r, 8) for r in range(8)]
    flat = sorted(x for b in blocks for x in b)
    assert flat[0][0] == 0 and flat[-1][1] == 1536 and len(flat) == 12
    assert all(a[1] == b[0] for a, b in zip(flat, flat[1:]))


def _oracle_fn(q, k, v, qb, kb, mask, causal, scale):
    return orc.attention_forward(q, k, v, qb, kb, mask, causal, scale)[0]


def _oracle_fwd_bwd(q, k, v, qb, kb, mask, causal, scale, do):
    o, lse, g = orc.attention_forward_backward(q, k, v, qb, kb, mask, causal, scale, do)
    return (o,) + tuple(g)


def test_shared_factor_flags():
    # alibi: factors per head, sharded by heads -> nothing shared
    assert shared_factor_flags(1, 50, (1, 8, 50, 2), (1, 8, 50, 2), 8) == (False, False)
    # swin: batch-broadcast factors, sharded by batch -> both shared
    assert shared_factor_flags(64, 24, (1, 8, 24, 16), (1, 8, 24, 16), 8) == (True, True)
    # pde: head-broadcast factors, 2 batch entries x 8 heads over 8 ranks -> shared within a batch entry
    assert shared_factor_flags(2, 8, (2, 8, 1, 5), (2, 8, 1, 5), 8) == (True, True)
    assert shared_factor_flags(2, 8, (2, 8, 1, 5), (2, 8, 1, 5), 2) == (False, False)
    assert shared_factor_flags(2, 8, None, None, 8) == (False, False)


def _worker(rank, world, port, q, k, v, qb, kb, want):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        pieces = sharded_attention(_oracle_fn, q, k, v, qb, kb, None, True, 0.3, rank=rank, world=world)
        full = gather_bh(pieces, *q.shape)
        # shards are independent problems: the assembled result equals the unsharded one bit for bit
        assert torch.equal(full, want)
        # forward + backward: the factor gradients of factors shared between ranks need the one sum across ranks
        g = torch.Generator().manual_seed(11)
        do = torch.randn(q.shape, generator=g)
        _, _, g_full = orc.attention_forward_backward(q, k, v, qb, kb, None, True, 0.3, do)
        res, dqb, dkb = sharded_forward_backward(_oracle_fwd_bwd, q, k, v, do, qb, kb, None, True, 0.3,
                                                 rank=rank, world=world)
        qs, ks = shared_factor_flags(q.shape[0], q.shape[2], qb.shape, kb.shape, world)
        # the batch-broadcast q-side factor is shared by the two ranks (one batch entry each); the head-broadcast
        # k-side factor is not: each rank holds every head of its batch entry
        assert (qs, ks) == (True, False)
        dqb, dkb = allreduce_shared_factor_grads(dqb, dkb, qs, ks)
        assert torch.allclose(dqb, g_full[3], atol=1e-5)
        assert torch.allclose(dkb[rank], g_full[4][rank], atol=1e-5) and not dkb[1 - rank].any()
        for (b, h0, h1), (o, dq, dk, dv) in res:
            assert torch.equal(dk, g_full[1][b:b + 1, :, h0:h1]) and torch.equal(dv, g_full[2][b:b + 1, :, h0:h1])
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
