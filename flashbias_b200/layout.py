"""Caller-side layout glue of the FlashBias call sites, fused into one pass.

The reference's call sites hold (B, H, S, D) tensors (often fp32) and run
``x.permute(0, 2, 1, 3).contiguous().half()`` -- Swin-V2 also ``F.normalize(q, dim=-1) * logit_scale`` -- on
each of q, k, v before every call (2_Vision_Transformer/swin_transformer_v2.py:194-199,
4_AlphaFold3/protenix/openfold_local/model/primitives.py:636-640).  ``prepare_bhsd`` does the cast, the
optional normalisation and the optional per-head scale in ONE kernel that reads the tensor where it lies
and writes a 16-bit tensor in the same (B, H, S, D) layout; the value returned is its (B, S, H, D) *view*,
which ``flash_bias_func`` takes as it is (the C ABI addresses batch, head and row through strides).
A 16-bit (B, H, S, D) tensor that needs neither normalisation nor scale needs no kernel at all:
``x.permute(0, 2, 1, 3)`` is already a valid argument.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib

__all__ = ["prepare_bhsd"]

_DT = {torch.float16: _lib.FB_DTYPE_F16, torch.bfloat16: _lib.FB_DTYPE_BF16, torch.float32: _lib.FB_DTYPE_F32}


def prepare_bhsd(x: torch.Tensor, dtype: torch.dtype = torch.float16, normalize: bool = False,
                 head_scale: Optional[torch.Tensor] = None, eps: float = 1e-12) -> torch.Tensor:
    """``x``: (B, H, S, D) CUDA tensor, any batch/head/row strides, rows contiguous, fp32/fp16/bf16.
    Returns the (B, S, H, D) view of a new ``dtype`` tensor holding ``normalize?(x) * head_scale[h]``."""
    assert x.dim() == 4 and x.is_cuda and x.stride(-1) == 1
    B, H, S, D = x.shape
    y = torch.empty((B, H, S, D), dtype=dtype, device=x.device)
    hs = None
    if head_scale is not None:
        hs = head_scale.detach().to(device=x.device, dtype=torch.float32).reshape(-1).contiguous()
        assert hs.numel() == H
    xs = (C.c_int64 * 3)(x.stride(0), x.stride(1), x.stride(2))
    ys = (C.c_int64 * 3)(y.stride(0), y.stride(1), y.stride(2))
    with torch.cuda.device(x.device):
        rc = _lib.load().fb_prepare_rows(x.data_ptr(), _DT[x.dtype], xs, y.data_ptr(), _DT[dtype], ys, B, H, S, D,
                                         1 if normalize else 0, hs.data_ptr() if hs is not None else None,
                                         float(eps), torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "fb_prepare_rows")
    return y.permute(0, 2, 1, 3)
