"""Forward + backward from pinned host buffers, with the copies overlapped with the kernels.

A caller whose tensors live in host memory pays three serial phases per call: inputs to the device,
the kernels, results back.  Every (batch, head) pair is an independent attention problem, so the work
is cut into chunks of heads (or of batch entries when the factors are shared over heads); chunk i+1
is copied in on one copy stream while chunk i computes, and the results of chunk i-1 go back on a
second copy stream.  Head chunks are strided slices of the (B, S, H, D) layout: they are moved with
2-D copies into the same positions of full-size device tensors, and the operator runs on views of
those (the C ABI takes strides, so no repacking).  The results are those of one call on the whole
tensors: a chunk is only ever a set of whole (batch, head) problems, and a factor gradient is never
split across chunks (the chunk dimension is chosen such that the factors are not shared along it; if
there is no such dimension the call runs as a single chunk).  o, dk and dv are bit-identical; dq and the
factor gradients are fp32 sums over key tiles whose order of addition is not fixed in either form.

Inputs and outputs are dictionaries of pinned host tensors in the operator's own layouts:
``q (B,Sq,H,D)``, ``k, v (B,Sk,H,D)``, ``q_bias / k_bias (B|1, S, H|1, R)`` (optional), ``do`` like ``q``;
outputs ``o, dq`` like ``q``, ``dk, dv`` like ``k``, ``dq_bias / dk_bias`` like the factors.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional, Tuple

import torch

from .flash_bias import flash_bias_backward, flash_bias_forward

__all__ = ["HostPipeline", "plan_chunks"]

_H2D, _D2H = 1, 2
_cudart = None


def _rt():
    global _cudart
    if _cudart is None:
        _cudart = C.CDLL("libcudart.so.12")
        _cudart.cudaMemcpy2DAsync.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t,
                                              C.c_int, C.c_void_p]
        _cudart.cudaMemcpy2DAsync.restype = C.c_int
    return _cudart


def _copy_heads(dst: torch.Tensor, src: torch.Tensor, h0: int, h1: int, kind: int, stream: torch.cuda.Stream):
    """Copy heads [h0, h1) of a (B, S, H, C) tensor between host and device.  `dst` and `src` are either both
    full-size (same shape: the slice goes to the same position) or one of them is the contiguous chunk
    (B, S, h1-h0, C)."""
    B, S, H, Cc = (src if src.shape[2] >= dst.shape[2] else dst).shape
    es = src.element_size()
    width = (h1 - h0) * Cc * es

    def base_and_pitch(t):
        if t.shape[2] == H and H != h1 - h0:
            return t.data_ptr() + h0 * Cc * es, H * Cc * es
        return t.data_ptr(), t.shape[2] * Cc * es
    dp, dpitch = base_and_pitch(dst)
    sp, spitch = base_and_pitch(src)
    rc = _rt().cudaMemcpy2DAsync(dp, dpitch, sp, spitch, width, B * S, kind, stream.cuda_stream)
    if rc != 0:
        raise RuntimeError(f"cudaMemcpy2DAsync failed: {rc}")


def plan_chunks(q_shape, q_bias_shape, k_bias_shape, in_bytes: int, chunks: int = 5, min_row_bytes: int = 512):
    """Host logic of the pipeline: along which dimension the work is cut and into which ranges.

    Returns (dim, ranges) with dim in {"head", "batch", "none"}.  The dimension is one the factors are not
    shared over, so that a factor gradient belongs to exactly one chunk; a chunk must carry at least ~4 MB of
    inputs to be worth its launches, and a head chunk -- a strided slice of the (B, S, H, D) layout, moved as a
    2-D copy -- must keep rows of at least `min_row_bytes` (short rows make the copy engine descriptor-bound:
    a few heads of head_dim 32 are 64..256-byte rows).
    """
    B, _, H, D = q_shape
    has_bias = q_bias_shape is not None
    per_head = (not has_bias) or (q_bias_shape[2] == H and k_bias_shape[2] == H)
    per_batch = (not has_bias) or (q_bias_shape[0] == B and k_bias_shape[0] == B)
    if per_head and H > 1:
        dim, n = "head", H
    elif per_batch and B > 1:
        dim, n = "batch", B
    else:
        dim, n = "none", 1
    chunks = max(1, min(chunks, n, in_bytes // (4 << 20)))
    if dim == "head":
        chunks = max(1, min(chunks, (H * D * 2) // max(min_row_bytes, 1)))
    if chunks == 1:
        return "none", [(0, n)]
    base, extra = divmod(n, chunks)
    ranges, lo = [], 0
    for c in range(chunks):
        hi = lo + base + (1 if c < extra else 0)
        ranges.append((lo, hi))
        lo = hi
    return dim, ranges


class HostPipeline:
    """Reusable device buffers and copy streams for ``run`` (one instance per problem shape)."""

    def __init__(self, host_in: Dict[str, torch.Tensor], device, chunks: int = 5):
        q, k = host_in["q"], host_in["k"]
        self.B, self.Sq, self.H, self.D = q.shape
        self.device = torch.device(device)
        qb, kb = host_in.get("q_bias"), host_in.get("k_bias")
        in_bytes = sum(t.numel() * t.element_size() for t in host_in.values() if t is not None)
        self.dim, self.ranges = plan_chunks(tuple(q.shape), None if qb is None else tuple(qb.shape),
                                            None if kb is None else tuple(kb.shape), in_bytes, chunks)
        self.dev = {name: torch.empty(t.shape, dtype=t.dtype, device=self.device)
                    for name, t in host_in.items() if t is not None}
        self.copy_in, self.copy_out = torch.cuda.Stream(self.device), torch.cuda.Stream(self.device)

    # ---- slices ---------------------------------------------------------------------------------
    def _view(self, t: Optional[torch.Tensor], lo: int, hi: int) -> Optional[torch.Tensor]:
        if t is None:
            return None
        if self.dim == "head":
            return t if t.shape[2] == 1 else t[:, :, lo:hi]
        if self.dim == "batch":
            return t if t.shape[0] == 1 else t[lo:hi]
        return t

    def _to_device(self, name: str, host: torch.Tensor, lo: int, hi: int, first: bool):
        dst = self.dev[name]
        shared = (self.dim == "head" and host.shape[2] == 1) or (self.dim == "batch" and host.shape[0] == 1)
        if self.dim == "none" or shared:
            if first:
                dst.copy_(host, non_blocking=True)
        elif self.dim == "batch":
            dst[lo:hi].copy_(host[lo:hi], non_blocking=True)
        else:
            _copy_heads(dst, host, lo, hi, _H2D, self.copy_in)

    def _to_host(self, host: torch.Tensor, chunk: torch.Tensor, lo: int, hi: int):
        if self.dim == "none":
            host.copy_(chunk, non_blocking=True)
        elif self.dim == "batch":
            host[lo:hi].copy_(chunk, non_blocking=True)
        else:
            _copy_heads(host, chunk, lo, hi, _D2H, self.copy_out)

    # ---- one forward + backward -----------------------------------------------------------------------
    def run(self, host_in: Dict[str, torch.Tensor], host_out: Dict[str, torch.Tensor], causal: bool,
            softmax_scale: Optional[float]):
        """Copies in, forward, backward, copies out; returns after everything has completed."""
        main = torch.cuda.current_stream(self.device)
        self.copy_in.wait_stream(main)
        self.copy_out.wait_stream(main)
        ready = []
        with torch.cuda.stream(self.copy_in):
            for i, (lo, hi) in enumerate(self.ranges):
                evs = []
                for group in (("q", "k", "v", "q_bias", "k_bias"), ("do",)):  # dO is only needed by the backward
                    for name in group:
                        if host_in.get(name) is not None:
                            self._to_device(name, host_in[name], lo, hi, i == 0)
                    ev = torch.cuda.Event()
                    ev.record()
                    evs.append(ev)
                ready.append(evs)
        keep = []  # chunk results stay referenced until their copies have completed
        d = self.dev

        def send_back(res, lo, hi):
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(self.copy_out):
                self.copy_out.wait_event(done)
                for name, t in res.items():
                    if t is not None:
                        self._to_host(host_out[name], t, lo, hi)

        for (lo, hi), (ev_fwd, ev_bwd) in zip(self.ranges, ready):
            main.wait_event(ev_fwd)
            q, k, v, do = (self._view(d[n], lo, hi) for n in ("q", "k", "v", "do"))
            qb, kb = self._view(d.get("q_bias"), lo, hi), self._view(d.get("k_bias"), lo, hi)
            o, lse, sc = flash_bias_forward(q, k, v, qb, kb, None, causal, softmax_scale)
            send_back({"o": o}, lo, hi)  # o leaves while the backward runs
            main.wait_event(ev_bwd)
            dq, dk, dv, dqb, dkb = flash_bias_backward(do, q, k, v, o, qb, kb, lse, None, causal, sc)
            res = {"dq": dq, "dk": dk, "dv": dv, "dq_bias": dqb, "dk_bias": dkb}
            send_back(res, lo, hi)
            keep.append((o, res))
        torch.cuda.synchronize(self.device)
        return keep[-1] if keep else None
