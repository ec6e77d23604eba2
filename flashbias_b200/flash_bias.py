"""``flash_bias_func`` -- the reference's operator on top of the B200 C ABI.

Mirrors ``FlashBiasFunc`` / ``flash_bias_func`` of the reference
(flash_bias/flash_bias_triton.py:1345-1405): same positional signature
``(q, k, v, q_bias=None, k_bias=None, mask=None, causal=False, softmax_scale=None)``, same layouts
((B, S, H, D) tensors, (B|1, S, H|1, R) factors, 4-D additive mask), same host-side checks and
messages (:1102-1127, :1206-1210, :1371), outputs as fresh tensors, inputs never mutated.

Differences, on purpose: gradients of factors that are broadcast over batch and/or heads are summed
over the broadcast dimensions (the reference indexes them with the un-expanded strides, :1227-1231);
a query row that sees no key yields 0 / -inf instead of NaN.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional

import torch

from . import _lib

__all__ = ["FlashBiasFunc", "flash_bias_func", "flash_bias_forward", "flash_bias_backward"]

_DT = {torch.float16: _lib.FB_DTYPE_F16, torch.bfloat16: _lib.FB_DTYPE_BF16, torch.float32: _lib.FB_DTYPE_F32}


def _strides_bhs(t: torch.Tensor):
    """(batch, head, row) element strides of a (B, S, H, C) tensor."""
    return _lib.I64x3(t.stride(0), t.stride(2), t.stride(1))


def _factor_strides(t: torch.Tensor):
    """As above with 0 for broadcast (size-1) batch/head dims."""
    return _lib.I64x3(0 if t.shape[0] == 1 else t.stride(0), 0 if t.shape[2] == 1 else t.stride(2), t.stride(1))


def _fill_common(p: _lib.FbParams, q, k, v, q_bias, k_bias, mask, causal, softmax_scale, flags):
    batch, seqlen_q, nheads, d = q.shape
    _, seqlen_k, _, _ = k.shape
    p.B, p.H, p.Sq, p.Sk, p.D = batch, nheads, seqlen_q, seqlen_k, d
    p.R = q_bias.shape[-1] if q_bias is not None else 0
    p.dtype = _DT[q.dtype]
    p.causal = 1 if causal else 0
    p.flags = flags
    p.softmax_scale = softmax_scale
    p.q, p.k, p.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    p.q_stride, p.k_stride, p.v_stride = _strides_bhs(q), _strides_bhs(k), _strides_bhs(v)
    if q_bias is not None:
        p.q_bias, p.k_bias = q_bias.data_ptr(), k_bias.data_ptr()
        p.q_bias_stride, p.k_bias_stride = _factor_strides(q_bias), _factor_strides(k_bias)
    if mask is not None:
        p.mask = mask.data_ptr()
        p.mask_dtype = _DT[mask.dtype]
        # (1, seqlen_k) is tested first, as in the reference (:1120-1123)
        p.mask_kind = _lib.FB_MASK_VECTOR if mask.shape[2] == 1 else _lib.FB_MASK_MATRIX
        p.mask_stride = _lib.I64x3(0 if mask.shape[0] == 1 else mask.stride(0),
                                   0 if mask.shape[1] == 1 else mask.stride(1),
                                   0 if mask.shape[2] == 1 else mask.stride(2))


def _check_inputs(q, k, v, q_bias, k_bias, mask):
    batch, seqlen_q, nheads, d = q.shape
    _, seqlen_k, _, _ = k.shape
    assert k.shape == (batch, seqlen_k, nheads, d)
    assert v.shape == (batch, seqlen_k, nheads, d)
    assert d <= 128, "FlashAttention only support head dimensions up to 128"
    assert q.dtype == k.dtype == v.dtype, "All tensors must have the same type"
    assert q.dtype in [torch.float16, torch.bfloat16], "Only support fp16 and bf16"
    assert q.is_cuda and k.is_cuda and v.is_cuda
    if (q_bias is None) != (k_bias is None):
        raise RuntimeError("q_bias and k_bias must be given together")
    if q_bias is not None:
        assert q_bias.dtype == k_bias.dtype == q.dtype, "All tensors must have the same type"
        assert q_bias.dim() == 4 and k_bias.dim() == 4
        rank = q_bias.shape[-1]
        assert k_bias.shape[-1] == rank
        assert q_bias.shape[0] in (1, batch) and q_bias.shape[2] in (1, nheads) and q_bias.shape[1] == seqlen_q
        assert k_bias.shape[0] in (1, batch) and k_bias.shape[2] in (1, nheads) and k_bias.shape[1] == seqlen_k
    if mask is not None:
        assert mask.dtype in [q.dtype, torch.float]
        assert mask.is_cuda
        assert mask.dim() == 4
        if mask.shape[2:] != (1, seqlen_k) and mask.shape[2:] != (seqlen_q, seqlen_k):
            raise RuntimeError("Last 2 dimensions of mask must be (1, seqlen_k) or (seqlen_q, seqlen_k)")
        assert mask.shape[0] in (1, batch) and mask.shape[1] in (1, nheads)


def _workspace(nbytes: int, device) -> Optional[torch.Tensor]:
    return torch.empty(nbytes, dtype=torch.uint8, device=device) if nbytes else None


def flash_bias_forward(q, k, v, q_bias=None, k_bias=None, mask=None, causal=False, softmax_scale=None, flags=0):
    """Forward launch (the role of ``_flash_attn_forward``, flash_bias_triton.py:1100-1194).

    Returns (o, lse, softmax_scale); lse is fp32 of shape (B, H, ceil(Sq/128)*128).
    """
    lib = _lib.load()
    _check_inputs(q, k, v, q_bias, k_bias, mask)
    batch, seqlen_q, nheads, d = q.shape
    softmax_scale = softmax_scale or 1.0 / math.sqrt(d)
    if mask is not None and mask.stride(-1) != 1:
        mask = mask.contiguous()
    seqlen_q_rounded = math.ceil(seqlen_q / 128) * 128
    lse = torch.empty((batch, nheads, seqlen_q_rounded), device=q.device, dtype=torch.float32)
    o = torch.empty_like(q)
    p = _lib.FbParams()
    _fill_common(p, q, k, v, q_bias, k_bias, mask, causal, float(softmax_scale), flags)
    p.o, p.o_stride = o.data_ptr(), _strides_bhs(o)
    p.lse, p.lse_stride_bh = lse.data_ptr(), seqlen_q_rounded
    with torch.cuda.device(q.device):
        ws = _workspace(lib.fb_fwd_workspace_bytes(C.byref(p)), q.device)
        if ws is not None:
            p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
        _lib.check(lib.fb_fwd(C.byref(p), torch.cuda.current_stream().cuda_stream), "fb_fwd")
    return o, lse, softmax_scale


def flash_bias_backward(do, q, k, v, o, q_bias, k_bias, lse, mask=None, causal=False, softmax_scale=None, flags=0):
    """Backward launches (the role of ``_flash_attn_backward``, flash_bias_triton.py:1197-1342).

    Returns (dq, dk, dv, dq_bias, dk_bias); factor gradients have the shape of the factors.
    """
    lib = _lib.load()
    if do.stride(-1) != 1:
        do = do.contiguous()
    batch, seqlen_q, nheads, d = q.shape
    assert d <= 128
    seqlen_q_rounded = math.ceil(seqlen_q / 128) * 128
    assert lse.shape == (batch, nheads, seqlen_q_rounded)
    assert q.stride(-1) == k.stride(-1) == v.stride(-1) == o.stride(-1) == 1
    softmax_scale = softmax_scale or 1.0 / math.sqrt(d)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    dq_bias = torch.empty_like(q_bias) if q_bias is not None else None
    dk_bias = torch.empty_like(k_bias) if k_bias is not None else None
    delta = torch.empty_like(lse)
    p = _lib.FbParams()
    _fill_common(p, q, k, v, q_bias, k_bias, mask, causal, float(softmax_scale), flags)
    p.o, p.o_stride = o.data_ptr(), _strides_bhs(o)
    p.lse, p.lse_stride_bh = lse.data_ptr(), seqlen_q_rounded
    p.dout, p.dout_stride = do.data_ptr(), _strides_bhs(do)
    p.delta = delta.data_ptr()
    p.dq, p.dk, p.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    p.dq_stride, p.dk_stride, p.dv_stride = _strides_bhs(dq), _strides_bhs(dk), _strides_bhs(dv)
    if q_bias is not None:
        p.dq_bias, p.dk_bias = dq_bias.data_ptr(), dk_bias.data_ptr()
        p.dq_bias_stride, p.dk_bias_stride = _strides_bhs(dq_bias), _strides_bhs(dk_bias)
    with torch.cuda.device(q.device):
        ws = _workspace(lib.fb_bwd_workspace_bytes(C.byref(p)), q.device)
        if ws is not None:
            p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
        stream = torch.cuda.current_stream().cuda_stream
        _lib.check(lib.fb_bwd_preprocess(C.byref(p), stream), "fb_bwd_preprocess")
        _lib.check(lib.fb_bwd(C.byref(p), stream), "fb_bwd")
    return dq, dk, dv, dq_bias, dk_bias


class FlashBiasFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, q_bias=None, k_bias=None, mask=None, causal=False, softmax_scale=None):
        """
        q: (batch_size, seqlen_q, nheads, headdim)
        k, v: (batch_size, seqlen_k, nheads, headdim)
        q_bias: (batch_size | 1, seqlen_q, nheads | 1, rankdim)
        k_bias: (batch_size | 1, seqlen_k, nheads | 1, rankdim)
        mask: optional, (batch | 1, nheads | 1, 1 | seqlen_q, seqlen_k), added to the logits.
        softmax_scale: multiplies q.k only; defaults to 1 / sqrt(headdim).
        """
        # Make sure that the last dimension is contiguous
        if q_bias is not None:
            q, k, v, q_bias, k_bias = [x if x.stride(-1) == 1 else x.contiguous() for x in [q, k, v, q_bias, k_bias]]
        else:
            q, k, v = [x if x.stride(-1) == 1 else x.contiguous() for x in [q, k, v]]
        o, lse, ctx.softmax_scale = flash_bias_forward(
            q, k, v, q_bias, k_bias, mask=mask, causal=causal, softmax_scale=softmax_scale)
        ctx.save_for_backward(q, k, v, o, q_bias, k_bias, lse, mask)
        ctx.causal = causal
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, q_bias, k_bias, lse, mask = ctx.saved_tensors
        assert not ctx.needs_input_grad[5], "FlashBias does not support mask gradient yet"
        with torch.inference_mode():
            dq, dk, dv, dq_bias, dk_bias = flash_bias_backward(
                do, q, k, v, o, q_bias, k_bias, lse, mask=mask, causal=ctx.causal, softmax_scale=ctx.softmax_scale)
        return dq, dk, dv, dq_bias, dk_bias, None, None, None


flash_bias_func = FlashBiasFunc.apply
