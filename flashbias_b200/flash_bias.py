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

__all__ = ["FlashBiasFunc", "flash_bias_func", "flash_bias_forward", "flash_bias_backward",
           "FlashBiasAlibiFunc", "flash_bias_alibi_func", "check_device_status"]

_DT = {torch.float16: _lib.FB_DTYPE_F16, torch.bfloat16: _lib.FB_DTYPE_BF16, torch.float32: _lib.FB_DTYPE_F32}


def _strides_bhs(t: torch.Tensor):
    """(batch, head, row) element strides of a (B, S, H, C) tensor (a tuple: ctypes converts it on assignment)."""
    sb, ss, sh, _ = t.stride()
    return (sb, sh, ss)


def _factor_strides(t: torch.Tensor):
    """As above with 0 for broadcast (size-1) batch/head dims."""
    sb, ss, sh, _ = t.stride()
    return (0 if t.shape[0] == 1 else sb, 0 if t.shape[2] == 1 else sh, ss)


_status = None
_status_ptr = 0        # address of the status word
_status_view = None    # ctypes view of it: reading a host word must not cost a tensor operation per call


def _status_word() -> torch.Tensor:
    """One int32 in pinned (device-visible) host memory: kernels store a device-side error code there, the host
    reads it without synchronising anything."""
    global _status, _status_ptr, _status_view
    if _status is None:
        _status = torch.zeros(1, dtype=torch.int32).pin_memory()
        _status_ptr = _status.data_ptr()
        _status_view = C.c_int32.from_address(_status_ptr)
    return _status


def check_device_status() -> None:
    """Raise if a kernel of an earlier call reported a device-side error (a bounded wait that expired, a factor
    that overflowed the 16-bit type); the results of that call are invalid.  Called at the start of every
    forward and backward; callers can also call it after a synchronisation point of their own."""
    if _status is None:
        return
    code = _status_view.value
    if code != 0:
        _status.zero_()
        raise RuntimeError(f"flashbias_b200: device-side error {code}: "
                           f"{_lib.load().fb_status_string(code).decode()} [{_lib.strerror(-10)}]")


_ws_cache = {}


def _fill_common(p: _lib.FbParams, q, k, v, q_bias, k_bias, mask, causal, softmax_scale, flags, alibi_slopes=None):
    batch, seqlen_q, nheads, d = q.shape
    _, seqlen_k, _, _ = k.shape
    p.B, p.H, p.Sq, p.Sk, p.D = batch, nheads, seqlen_q, seqlen_k, d
    p.R = q_bias.shape[-1] if q_bias is not None else 0
    p.dtype = _DT[q.dtype]
    p.causal = 1 if causal else 0
    p.flags = flags
    p.softmax_scale = softmax_scale
    if _status is None:
        _status_word()
    p.status = _status_ptr
    if alibi_slopes is not None:
        p.alibi_slopes = alibi_slopes.data_ptr()
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
        p.mask_stride = (0 if mask.shape[0] == 1 else mask.stride(0),
                         0 if mask.shape[1] == 1 else mask.stride(1),
                         0 if mask.shape[2] == 1 else mask.stride(2))
        # a mask with fewer batch entries than q is read periodically (entry b % n): Swin's shift mask
        p.mask_batch_period = mask.shape[0] if 1 < mask.shape[0] < batch else 0


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
        # the reference expands the mask over batch and heads (:1128); a mask of n batch entries with n
        # dividing the batch is also taken and read periodically, which is what Swin's repeat() produces
        assert (mask.shape[0] in (1, batch) or batch % mask.shape[0] == 0) and mask.shape[1] in (1, nheads)


def _raw_stream(device) -> int:
    """cudaStream_t of torch's current stream on `device`, as an integer."""
    return torch._C._cuda_getCurrentRawStream(device.index)


class _on_device:
    """`with` block that makes `device` current; does nothing when it already is (the usual case)."""

    def __init__(self, device):
        self.ctx = None if torch.cuda.current_device() == device.index else torch.cuda.device(device)

    def __enter__(self):
        if self.ctx is not None:
            self.ctx.__enter__()

    def __exit__(self, *exc):
        if self.ctx is not None:
            self.ctx.__exit__(*exc)


def _workspace(nbytes: int, device, stream: int) -> Optional[torch.Tensor]:
    """Scratch for one call.  One buffer per (device, stream) is kept and grown on demand: calls on a stream
    are ordered, so the next call may overwrite it, and no allocation happens in the steady state."""
    if not nbytes:
        return None
    key = (device.index, stream)
    ws = _ws_cache.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _ws_cache[key] = ws
    return ws


def flash_bias_forward(q, k, v, q_bias=None, k_bias=None, mask=None, causal=False, softmax_scale=None, flags=0,
                       alibi_slopes=None):
    """Forward launch (the role of ``_flash_attn_forward``, flash_bias_triton.py:1100-1194).

    Returns (o, lse, softmax_scale); lse is fp32 of shape (B, H, ceil(Sq/128)*128).
    """
    lib = _lib.load()
    check_device_status()
    _check_inputs(q, k, v, q_bias, k_bias, mask)
    batch, seqlen_q, nheads, d = q.shape
    softmax_scale = softmax_scale or 1.0 / math.sqrt(d)
    if mask is not None and mask.stride(-1) != 1:
        mask = mask.contiguous()
    seqlen_q_rounded = math.ceil(seqlen_q / 128) * 128
    lse = torch.empty((batch, nheads, seqlen_q_rounded), device=q.device, dtype=torch.float32)
    o = torch.empty_like(q)
    p = _lib.FbParams()
    _fill_common(p, q, k, v, q_bias, k_bias, mask, causal, float(softmax_scale), flags, alibi_slopes)
    p.o, p.o_stride = o.data_ptr(), _strides_bhs(o)
    p.lse, p.lse_stride_bh = lse.data_ptr(), seqlen_q_rounded
    with _on_device(q.device):
        stream = _raw_stream(q.device)
        ws = _workspace(lib.fb_fwd_workspace_bytes(C.byref(p)), q.device, stream)
        if ws is not None:
            p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
        _lib.check(lib.fb_fwd(C.byref(p), stream), "fb_fwd")
    return o, lse, softmax_scale


def flash_bias_backward(do, q, k, v, o, q_bias, k_bias, lse, mask=None, causal=False, softmax_scale=None, flags=0,
                        alibi_slopes=None):
    """Backward launches (the role of ``_flash_attn_backward``, flash_bias_triton.py:1197-1342).

    Returns (dq, dk, dv, dq_bias, dk_bias); factor gradients have the shape of the factors.
    """
    lib = _lib.load()
    check_device_status()
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
    _fill_common(p, q, k, v, q_bias, k_bias, mask, causal, float(softmax_scale), flags, alibi_slopes)
    p.o, p.o_stride = o.data_ptr(), _strides_bhs(o)
    p.lse, p.lse_stride_bh = lse.data_ptr(), seqlen_q_rounded
    p.dout, p.dout_stride = do.data_ptr(), _strides_bhs(do)
    p.delta = delta.data_ptr()
    p.dq, p.dk, p.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    p.dq_stride, p.dk_stride, p.dv_stride = _strides_bhs(dq), _strides_bhs(dk), _strides_bhs(dv)
    if q_bias is not None:
        p.dq_bias, p.dk_bias = dq_bias.data_ptr(), dk_bias.data_ptr()
        p.dq_bias_stride, p.dk_bias_stride = _strides_bhs(dq_bias), _strides_bhs(dk_bias)
    with _on_device(q.device):
        stream = _raw_stream(q.device)
        ws = _workspace(lib.fb_bwd_workspace_bytes(C.byref(p)), q.device, stream)
        if ws is not None:
            p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
        _lib.check(lib.fb_bwd_preprocess(C.byref(p), stream), "fb_bwd_preprocess")
        _lib.check(lib.fb_bwd(C.byref(p), stream), "fb_bwd")
    return dq, dk, dv, dq_bias, dk_bias


def _narrow_expanded(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """A factor passed as an expanded view (size > 1, stride 0 on batch or heads) is a broadcast factor: hand the
    library the size-1 view, so that its gradient is the fp32 sum over the broadcast dimension."""
    if t is None:
        return None
    for dim in (0, 2):
        if t.shape[dim] > 1 and t.stride(dim) == 0:
            t = t.narrow(dim, 0, 1)
    return t


def _widen_grad(g: Optional[torch.Tensor], shape) -> Optional[torch.Tensor]:
    """Gradient for an input that was an expanded view: autograd sums the gradient over the expanded
    dimension, so the summed gradient goes into entry 0 and the other entries are zero."""
    if g is None or tuple(g.shape) == tuple(shape):
        return g
    full = torch.zeros(shape, dtype=g.dtype, device=g.device)
    view = full
    for dim in (0, 2):
        if g.shape[dim] != shape[dim]:
            view = view.narrow(dim, 0, 1)
    view.copy_(g)
    return full


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
        ctx.factor_shapes = (None if q_bias is None else tuple(q_bias.shape),
                             None if k_bias is None else tuple(k_bias.shape))
        q_bias, k_bias = _narrow_expanded(q_bias), _narrow_expanded(k_bias)
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
            dq_bias = _widen_grad(dq_bias, ctx.factor_shapes[0])
            dk_bias = _widen_grad(dk_bias, ctx.factor_shapes[1])
        return dq, dk, dv, dq_bias, dk_bias, None, None, None


flash_bias_func = FlashBiasFunc.apply


class FlashBiasAlibiFunc(torch.autograd.Function):
    """Attention with the ALiBi bias ``slopes[h] * (j - i)`` generated inside the kernels.

    The reference's language-model call site builds this bias as rank-2 factors from the positions and the
    per-head slopes (1_Language_Model/attention_with_alibi_bias.py:47-52) and feeds them to
    ``flash_bias_func``; here the slopes go in directly, the positions never exist as tensors and are never
    rounded to 16 bits.  ``slopes`` is an fp32 tensor of ``nheads`` values, a constant (the reference
    registers it as a buffer): it gets no gradient.
    """

    @staticmethod
    def forward(ctx, q, k, v, slopes, causal=True, softmax_scale=None):
        q, k, v = [x if x.stride(-1) == 1 else x.contiguous() for x in [q, k, v]]
        slopes = slopes.detach().to(device=q.device, dtype=torch.float32).reshape(-1).contiguous()
        assert slopes.numel() == q.shape[2], "one slope per head"
        o, lse, ctx.softmax_scale = flash_bias_forward(q, k, v, causal=causal, softmax_scale=softmax_scale,
                                                       alibi_slopes=slopes)
        ctx.save_for_backward(q, k, v, o, lse, slopes)
        ctx.causal = causal
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, slopes = ctx.saved_tensors
        with torch.inference_mode():
            dq, dk, dv, _, _ = flash_bias_backward(do, q, k, v, o, None, None, lse, causal=ctx.causal,
                                                   softmax_scale=ctx.softmax_scale, alibi_slopes=slopes)
        return dq, dk, dv, None, None, None


flash_bias_alibi_func = FlashBiasAlibiFunc.apply
