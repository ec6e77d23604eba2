"""Seeded synthetic inputs for the five benchmark workloads of the FlashBias path.

Every tensor is drawn on the CPU in fp32 from ``torch.Generator().manual_seed(seed)``
with ``seed = 1000 * workload + k`` (k: 0 q, 1 k, 2 v, 3 dO, 4+ factor sources) and
then rounded once to the run dtype, so the CPU checker and the CUDA kernels consume
bit-identical values.  The public workloads these stand in for (ImageNet/Swin
checkpoints, car-design meshes, PDB structures) are not reproduced; only their
shapes and value distributions are.

Workloads (shapes are the full-size defaults; every generator accepts smaller
sizes for tests):

* ``generic``   B2 H4 S1024 D32 R8, non-causal, i.i.d. N(0,1) factors, fp16.
  Shape of the reference's own benchmark (flash_bias/config.py:11).
* ``alibi``     B1 H50 S8192 D32 R2, causal, bf16.  ALiBi as an exact rank-2 bias
  ``m_h (j - i)`` with ``q_bias[i] = [-m_h i, 1]``, ``k_bias[j] = [1, m_h j]``,
  ``m_h = 2^(-8(h+1)/H)`` (slopes as in 1_Language_Model/attention_with_alibi_bias.py:8-15).
* ``swin``      B4096 H24 S256 (16x16 window) D32 R16, non-causal, bf16.  Bias table from a
  seeded 2-layer MLP over log-spaced relative coordinates (the construction of
  2_Vision_Transformer/swin_transformer_v2.py:98-131), factorised per head by
  truncated SVD; factors are batch-broadcast.
* ``pde``       B2 H8 S32768 D64 R5, non-causal, bf16.  ``-alpha |x_i - x_j|^2`` for points
  uniform in the unit cube as an exact rank-5 bias; factors are head-broadcast.
* ``pairformer`` B1 H16 S1536 D32 R32, non-causal, bf16.  A (S,S,128) pair representation
  projected to a per-head bias and factorised per head by truncated SVD.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

__all__ = ["Workload", "make_workload", "make_device_workload", "WORKLOADS", "flops_fwd", "flops_bwd",
           "attended_pairs", "alibi_slopes", "swin_shift_mask"]


@dataclass
class Workload:
    name: str
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    q_bias: torch.Tensor
    k_bias: torch.Tensor
    do: torch.Tensor
    causal: bool
    softmax_scale: float
    dtype: torch.dtype

    @property
    def shape(self):
        B, S, H, D = self.q.shape
        return dict(B=B, H=H, Sq=S, Sk=self.k.shape[1], D=D, R=self.q_bias.shape[-1])

    def to(self, device):
        return Workload(self.name, *(t.to(device) for t in
                                     (self.q, self.k, self.v, self.q_bias, self.k_bias, self.do)),
                        self.causal, self.softmax_scale, self.dtype)


def _randn(seed, shape):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g, dtype=torch.float32)


def _rand(seed, shape):
    g = torch.Generator().manual_seed(seed)
    return torch.rand(shape, generator=g, dtype=torch.float32)


def _qkvdo(cfg, B, S, H, D):
    return tuple(_randn(1000 * cfg + i, (B, S, H, D)) for i in range(4))


def _svd_factors(bias_hqk: torch.Tensor, rank: int):
    """(H,Sq,Sk) table -> q_bias (1,Sq,H,R) = U sqrt(S), k_bias (1,Sk,H,R) = V sqrt(S)."""
    U, S, Vh = torch.linalg.svd(bias_hqk.double(), full_matrices=False)
    rs = S[:, :rank].sqrt()
    qb = (U[:, :, :rank] * rs[:, None, :]).permute(1, 0, 2).unsqueeze(0)
    kb = (Vh[:, :rank, :].transpose(1, 2) * rs[:, None, :]).permute(1, 0, 2).unsqueeze(0)
    return qb.float().contiguous(), kb.float().contiguous()


def _generic_factors(B=2, H=4, S=1024, D=32, R=8, **_):
    return _randn(1004, (B, S, H, R)), _randn(1005, (B, S, H, R))


def _generic(B=2, H=4, S=1024, D=32, R=8, dtype=torch.float16, causal=False):
    q, k, v, do = _qkvdo(1, B, S, H, D)
    qb, kb = _generic_factors(B, H, S, D, R)
    return "generic", q, k, v, qb, kb, do, causal, 1.0 / math.sqrt(D), dtype


def alibi_slopes(H: int) -> torch.Tensor:
    """m_h = 2^(-8(h+1)/H) (1_Language_Model/attention_with_alibi_bias.py:8-15)."""
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=torch.float32)


def _alibi_factors(B=1, H=50, S=8192, D=32, **_):
    m = alibi_slopes(H)
    pos = torch.arange(S, dtype=torch.float32)
    qb = torch.stack([-(m[None, :] * pos[:, None]), torch.ones(S, H)], dim=-1).unsqueeze(0)
    kb = torch.stack([torch.ones(S, H), m[None, :] * pos[:, None]], dim=-1).unsqueeze(0)
    return qb.contiguous(), kb.contiguous()


def _alibi(B=1, H=50, S=8192, D=32, dtype=torch.bfloat16):
    q, k, v, do = _qkvdo(2, B, S, H, D)
    qb, kb = _alibi_factors(B, H, S, D)
    return "alibi", q, k, v, qb, kb, do, True, 1.0 / math.sqrt(D), dtype


def _swin_table(window: int, H: int, hidden: int = 512) -> torch.Tensor:
    """(H, N, N) relative-position bias of one window from a seeded MLP."""
    g = torch.Generator().manual_seed(3004)
    w1 = (torch.rand((hidden, 2), generator=g) * 2 - 1) / math.sqrt(2.0)
    b1 = (torch.rand((hidden,), generator=g) * 2 - 1) / math.sqrt(2.0)
    w2 = (torch.rand((H, hidden), generator=g) * 2 - 1) / math.sqrt(hidden)
    rel = torch.arange(-(window - 1), window, dtype=torch.float32)
    table = torch.stack(torch.meshgrid(rel, rel, indexing="ij"), dim=-1) / max(window - 1, 1) * 8.0
    table = torch.sign(table) * torch.log2(table.abs() + 1.0) / math.log2(8.0)
    feat = torch.relu(table.reshape(-1, 2) @ w1.t() + b1) @ w2.t()  # ((2w-1)^2, H)
    ys, xs = torch.meshgrid(torch.arange(window), torch.arange(window), indexing="ij")
    ys, xs = ys.flatten(), xs.flatten()
    dy = ys[:, None] - ys[None, :] + window - 1
    dx = xs[:, None] - xs[None, :] + window - 1
    idx = dy * (2 * window - 1) + dx
    return feat[idx.reshape(-1)].reshape(window * window, window * window, H).permute(2, 0, 1).contiguous()


def swin_shift_mask(window: int = 16, grid: int = 8) -> torch.Tensor:
    """(grid*grid, 1, N, N) fp32 additive mask of a shifted-window block, N = window*window: 0 where two tokens
    of a window come from the same image region, -100 elsewhere (the reference's call site builds it from the
    region map of the cyclically shifted image, 2_Vision_Transformer/swin_transformer_v2.py:189-192, :260-283).
    With a shift of half a window only the windows of the last row and column of the window grid straddle
    regions; the mask of batch entry b is entry b % (grid*grid)."""
    shift = window // 2
    ys, xs = torch.meshgrid(torch.arange(window), torch.arange(window), indexing="ij")
    out = torch.zeros(grid * grid, 1, window * window, window * window)
    for wy in range(grid):
        for wx in range(grid):
            region = (2 * ((ys >= window - shift) & (wy == grid - 1)) + ((xs >= window - shift) & (wx == grid - 1))).flatten()
            out[wy * grid + wx, 0] = torch.where(region[:, None] == region[None, :], 0.0, -100.0)
    return out


def _swin_factors(B=4096, H=24, window=16, D=32, R=16, **_):
    return _svd_factors(_swin_table(window, H), R)


def _swin(B=4096, H=24, window=16, D=32, R=16, dtype=torch.bfloat16):
    S = window * window
    q, k, v, do = _qkvdo(3, B, S, H, D)
    qb, kb = _swin_factors(B, H, window, D, R)
    return "swin", q, k, v, qb, kb, do, False, 1.0 / math.sqrt(D), dtype


def _pde_factors(B=2, H=8, S=32768, D=64, alpha=4.0, **_):
    x = _rand(4004, (B, S, 3))
    n2 = (x * x).sum(-1, keepdim=True)
    one = torch.ones_like(n2)
    qb = torch.cat([-alpha * n2, 2 * alpha * x, one], dim=-1).unsqueeze(2)   # (B,S,1,5)
    kb = torch.cat([one, x, -alpha * n2], dim=-1).unsqueeze(2)
    return qb.contiguous(), kb.contiguous()


def _pde(B=2, H=8, S=32768, D=64, alpha=4.0, dtype=torch.bfloat16):
    q, k, v, do = _qkvdo(4, B, S, H, D)
    qb, kb = _pde_factors(B, H, S, D, alpha)
    return "pde", q, k, v, qb, kb, do, False, 1.0 / math.sqrt(D), dtype


def _pairformer_factors(B=1, H=16, S=1536, D=32, R=32, C=128, **_):
    z = _randn(5004, (S, S, C))
    w = _randn(5005, (H, C)) / math.sqrt(C)
    bias = torch.einsum("ijc,hc->hij", z, w)
    return _svd_factors(bias, R)


def _pairformer(B=1, H=16, S=1536, D=32, R=32, C=128, dtype=torch.bfloat16):
    q, k, v, do = _qkvdo(5, B, S, H, D)
    qb, kb = _pairformer_factors(B, H, S, D, R, C)
    return "pairformer", q, k, v, qb, kb, do, False, 1.0 / math.sqrt(D), dtype


WORKLOADS = {"generic": _generic, "alibi": _alibi, "swin": _swin, "pde": _pde, "pairformer": _pairformer}
_FACTORS = {"generic": _generic_factors, "alibi": _alibi_factors, "swin": _swin_factors, "pde": _pde_factors,
            "pairformer": _pairformer_factors}
_META = {"generic": (torch.float16, False), "alibi": (torch.bfloat16, True), "swin": (torch.bfloat16, False),
         "pde": (torch.bfloat16, False), "pairformer": (torch.bfloat16, False)}


def make_workload(name: str, **sizes) -> Workload:
    """Build one workload on the CPU; all tensors are rounded once to the run dtype."""
    nm, q, k, v, qb, kb, do, causal, scale, dtype = WORKLOADS[name](**sizes)
    cast = lambda t: t.to(dtype).contiguous()
    return Workload(nm, cast(q), cast(k), cast(v), cast(qb), cast(kb), cast(do), causal, scale, dtype)


def make_device_workload(name: str, device, seed: int = 0, **sizes) -> Workload:
    """Timing-only variant of ``make_workload``: the factors are the seeded CPU ones, q/k/v/dO are drawn N(0,1)
    on the device (not bit-identical to the CPU-seeded tensors, which a timing run does not need), so that the
    large workloads do not spend a minute in the host generator."""
    dtype, causal = _META[name]
    qb, kb = _FACTORS[name](**sizes)
    B, H, D = sizes.get("B", qb.shape[0]), sizes["H"], sizes["D"]
    S = qb.shape[1]
    g = torch.Generator(device=device).manual_seed(seed)
    q, k, v, do = (torch.randn((B, S, H, D), generator=g, device=device, dtype=torch.float32).to(dtype)
                   for _ in range(4))
    return Workload(name, q, k, v, qb.to(dtype).to(device), kb.to(dtype).to(device), do, causal,
                    1.0 / math.sqrt(D), dtype)


def attended_pairs(B, H, Sq, Sk, causal) -> int:
    """Number of (query, key) pairs attended: B*H*Sq*Sk, or the top-left causal triangle."""
    if not causal:
        return B * H * Sq * Sk
    per = sum(min(i + 1, Sk) for i in range(Sq)) if Sq != Sk else Sq * (Sq + 1) // 2
    return B * H * per


def flops_fwd(B, H, Sq, Sk, D, R, causal) -> float:
    """T*(4D + 2R): logits over head_dim+rank and P.V, 2 flop per MAC."""
    return attended_pairs(B, H, Sq, Sk, causal) * (4.0 * D + 2.0 * R)


def flops_bwd(B, H, Sq, Sk, D, R, causal) -> float:
    """T*(10D + 6R): logit recompute, dV, dP, dQ|dq_bias, dK|dk_bias."""
    return attended_pairs(B, H, Sq, Sk, causal) * (10.0 * D + 6.0 * R)
