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

__all__ = ["shard_ranges", "bh_segments", "bh_slabs", "sharded_attention", "sharded_forward_backward", "shared_factor_flags",
           "allreduce_shared_factor_grads", "shard_query_blocks", "gather_bh"]


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


def bh_slabs(B: int, H: int, rank: int, world: int) -> List[Tuple[int, int, int, int]]:
    """This rank's range as (b0, b1, h0, h1) slabs: runs of whole batch entries are merged into one slab (all
    heads), a partially owned batch entry stays a slab of its own (one batch entry, a range of heads).  One
    operator call per slab."""
    slabs: List[Tuple[int, int, int, int]] = []
    for (b, h0, h1) in bh_segments(B, H, rank, world):
        if h0 == 0 and h1 == H and slabs and slabs[-1][2] == 0 and slabs[-1][3] == H and slabs[-1][1] == b:
            slabs[-1] = (slabs[-1][0], b + 1, 0, H)
        else:
            slabs.append((b, b + 1, h0, h1))
    return slabs


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


def shared_factor_flags(B: int, H: int, q_bias_shape, k_bias_shape, world: int) -> Tuple[bool, bool]:
    """Whether the q-side / k-side factor is shared between ranks under the (batch, head) partition, i.e.
    whether its gradient needs a sum across ranks.  A factor with its own slice per (batch, head) never is; a
    factor broadcast over batch and/or heads is as soon as two ranks hold pairs that map to the same slice."""
    def shared(shape) -> bool:
        if shape is None or world == 1:
            return False
        owners = {}
        for r in range(world):
            for (b, h0, h1) in bh_segments(B, H, r, world):
                for h in range(h0, h1):
                    key = (b if shape[0] > 1 else 0, h if shape[2] > 1 else 0)
                    if owners.setdefault(key, r) != r:
                        return True
        return False
    return shared(q_bias_shape), shared(k_bias_shape)


def sharded_forward_backward(fwd_bwd: Callable, q, k, v, do, q_bias=None, k_bias=None, mask=None, causal=False,
                             softmax_scale=None, *, rank: int, world: int):
    """Forward + backward of this rank's (batch, head) pieces.

    `fwd_bwd(q, k, v, q_bias, k_bias, mask, causal, softmax_scale, do)` returns (o, dq, dk, dv, dq_bias,
    dk_bias) for the tensors it is given.  Returns [((b, h0, h1), results), ...] and fp32 partial sums of the
    factor gradients in the shape of the full factors (zeros where this rank holds nothing), or None without
    factors.  A factor slice shared by several of this rank's pieces accumulates here; slices shared between
    ranks still need ``allreduce_shared_factor_grads``.
    """
    B, _, H, _ = q.shape
    out = []
    dqb = torch.zeros(q_bias.shape, dtype=torch.float32, device=q_bias.device) if q_bias is not None else None
    dkb = torch.zeros(k_bias.shape, dtype=torch.float32, device=k_bias.device) if k_bias is not None else None
    for (b, h0, h1) in bh_segments(B, H, rank, world):
        res = fwd_bwd(_slice_bh(q, b, h0, h1, 2), _slice_bh(k, b, h0, h1, 2), _slice_bh(v, b, h0, h1, 2),
                      _slice_bh(q_bias, b, h0, h1, 2), _slice_bh(k_bias, b, h0, h1, 2),
                      _slice_bh(mask, b, h0, h1, 1), causal, softmax_scale, _slice_bh(do, b, h0, h1, 2))
        out.append(((b, h0, h1), res[:4]))
        if q_bias is not None:
            _slice_bh(dqb, b, h0, h1, 2).add_(res[4].float())
            _slice_bh(dkb, b, h0, h1, 2).add_(res[5].float())
    return out, dqb, dkb


def allreduce_shared_factor_grads(dqb: Optional[torch.Tensor], dkb: Optional[torch.Tensor], q_shared: bool,
                                  k_shared: bool, group=None):
    """The one exchange step of the partition: fp32 sum across ranks of the gradient of a factor that ranks
    share (a few S*R floats).  It runs after the kernels, outside them; factors that are not shared are left
    alone, and their rows belonging to other ranks stay zero."""
    import torch.distributed as dist
    if q_shared and dqb is not None:
        dist.all_reduce(dqb, group=group)
    if k_shared and dkb is not None:
        dist.all_reduce(dkb, group=group)
    return dqb, dkb


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
