"""Partitioning of the FlashBias path across the GPUs of one box.

Every (batch, head) pair is an independent attention problem, so the path shards with no exchange
step: each rank takes a contiguous range of the flattened (batch, head) index and calls the operator
on views of the inputs (the C ABI takes strides, so head slices need no copy).  For a single long
sequence the forward can also be split over blocks of query rows with K, V and k_bias replicated.

The helpers here are host logic only; they take the attention callable as an argument, which is
``flash_bias_func`` on a GPU rank.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch

__all__ = ["shard_ranges", "bh_segments", "sharded_attention", "shard_query_blocks", "gather_bh"]


def shard_ranges(n: int, world: int) -> List[Tuple[int, int]]:
    """Split range(n) into `world` contiguous, near-equal ranges (the first n % world get one extra)."""
    if world <= 0:
        raise ValueError("world must be positive")
    base, extra = divmod(n, world)
    out, start = [], 0
    for r in range(world):
        stop = start + base + (1 if r < extra else 0)
        out.append((start, stop))
        start = stop
    return out


def bh_segments(B: int, H: int, rank: int, world: int) -> List[Tuple[int, int, int]]:
    """(batch, head_start, head_stop) pieces of this rank's range of the flattened (batch, head) index."""
    lo, hi = shard_ranges(B * H, world)[rank]
    segs = []
    while lo < hi:
        b, h0 = divmod(lo, H)
        h1 = min(H, h0 + (hi - lo))
        segs.append((b, h0, h1))
        lo += h1 - h0
    return segs


def _slice_bh(t: Optional[torch.Tensor], b: int, h0: int, h1: int, head_dim: int) -> Optional[torch.Tensor]:
    if t is None:
        return None
    bs = slice(0, 1) if t.shape[0] == 1 else slice(b, b + 1)
    hs = slice(0, 1) if t.shape[head_dim] == 1 else slice(h0, h1)
    idx = [slice(None)] * t.dim()
    idx[0], idx[head_dim] = bs, hs
    return t[tuple(idx)]


def sharded_attention(fn: Callable, q, k, v, q_bias=None, k_bias=None, mask=None, causal=False, softmax_scale=None,
                      *, rank: int, world: int):
    """Run `fn` on this rank's (batch, head) pieces.  Returns [((b, h0, h1), output), ...]."""
    B, _, H, _ = q.shape
    out = []
    for (b, h0, h1) in bh_segments(B, H, rank, world):
        o = fn(_slice_bh(q, b, h0, h1, 2), _slice_bh(k, b, h0, h1, 2), _slice_bh(v, b, h0, h1, 2),
               _slice_bh(q_bias, b, h0, h1, 2), _slice_bh(k_bias, b, h0, h1, 2), _slice_bh(mask, b, h0, h1, 1),
               causal, softmax_scale)
        out.append(((b, h0, h1), o))
    return out


def shard_query_blocks(Sq: int, rank: int, world: int, block: int = 128) -> List[Tuple[int, int]]:
    """Query-row ranges of this rank when a single sequence is dealt out in blocks of `block` rows,
    round-robin (balances causal work).  Forward only needs K/V replicated; no collective."""
    nblk = (Sq + block - 1) // block
    return [(i * block, min(Sq, (i + 1) * block)) for i in range(rank, nblk, world)]


def gather_bh(pieces: Sequence[Tuple[Tuple[int, int, int], torch.Tensor]], B: int, Sq: int, H: int, D: int,
              group=None) -> torch.Tensor:
    """Assemble the full (B, Sq, H, D) output from every rank's pieces (all_gather_object; for tests
    and small results -- production callers keep the shards where they are)."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    bucket = [None] * world
    dist.all_gather_object(bucket, [(seg, o.detach().cpu()) for seg, o in pieces], group=group)
    ref = pieces[0][1] if pieces else None
    full = torch.empty(B, Sq, H, D, dtype=ref.dtype if ref is not None else torch.float32)
    for rank_pieces in bucket:
        for (b, h0, h1), o in rank_pieces:
            full[b:b + 1, :, h0:h1] = o
    return full
