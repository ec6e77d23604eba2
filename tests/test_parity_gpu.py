"""Parity of the CUDA path (through the C ABI / flash_bias_func) with the CPU checker and with the
golden vectors produced by the reference's own naive attention."""
import math

import pytest
import torch

from flashbias_b200 import flash_bias_func
from flashbias_b200 import _lib
from flashbias_b200.flash_bias import flash_bias_backward, flash_bias_forward
from flashbias_b200.workloads import make_workload
from oracle import flashbias_oracle as orc
from tests.helpers import check_close, golden_names, load_golden

pytestmark = pytest.mark.gpu

GRADS = ("dq", "dk", "dv", "dq_bias", "dk_bias")


def _run_cuda(ins, case, dtype, flags=0):
    dev = "cuda"
    t = {k: v.to(dtype).to(dev) for k, v in ins.items() if k != "mask"}
    mask = ins["mask"].to(dev) if "mask" in ins else None  # fp32 mask
    o, lse, sc = flash_bias_forward(t["q"], t["k"], t["v"], t.get("q_bias"), t.get("k_bias"), mask,
                                    case["causal"], case["scale"], flags=flags)
    grads = flash_bias_backward(t["do"], t["q"], t["k"], t["v"], o, t.get("q_bias"), t.get("k_bias"), lse, mask,
                                case["causal"], sc, flags=flags)
    torch.cuda.synchronize()
    return o, lse, grads


@pytest.mark.parametrize("flags", [0, _lib.FB_FLAG_FORCE_GENERAL], ids=["default", "general"])
@pytest.mark.parametrize("name", golden_names())
def test_golden(name, flags):
    """Golden vectors of the reference's naive attention: edge shapes (ragged, cross-attention,
    causal with Sq != Sk, masks, broadcast factors, no bias, head_dim 16/24/64/128)."""
    case, ins, ref = load_golden(name)
    dtype = case["dtype"]
    o, lse, grads = _run_cuda(ins, case, dtype, flags)
    check_close(f"{name}/o", o, ref["o"], dtype)
    _, lse_ref = orc.attention_forward(ins["q"], ins["k"], ins["v"], ins.get("q_bias"), ins.get("k_bias"),
                                       ins.get("mask"), case["causal"], case["scale"])
    got = lse[:, :, :case["Sq"]].float().cpu()
    assert (got - lse_ref).abs().max().item() < 2e-2
    # Gradients, strict gate: against the checker's backward fed with the stored 16-bit o, which is what
    # the reference's backward consumes too (delta = rowsum(o * do), flash_bias_triton.py:384-400).
    g_ref = orc.attention_backward(ins["do"], ins["q"], ins["k"], ins["v"], o.float().cpu(), lse_ref,
                                   ins.get("q_bias"), ins.get("k_bias"), ins.get("mask"), case["causal"],
                                   case["scale"])
    for key, g, want in zip(GRADS, grads, g_ref):
        if want is not None:
            check_close(f"{name}/{key}", g, want, dtype)
    # Gradients against the golden autograd values (which differentiate through an unrounded o): the same
    # max-abs bound, and a relative-L2 bound widened by the rounding of o that enters delta.
    for key, g in zip(GRADS, grads):
        if key in ref:
            check_close(f"{name}/{key}/golden", g, ref[key], dtype, rel_l2_tol=2.5e-3)


SMALL = {
    "generic": dict(B=2, H=4, S=1024, D=32, R=8),
    "alibi": dict(B=1, H=4, S=1024, D=32),
    "swin": dict(B=8, H=24, window=16, D=32, R=16),
    "pde": dict(B=1, H=2, S=2048, D=64),
    "pairformer": dict(B=1, H=4, S=512, D=32, R=32),
}


@pytest.mark.parametrize("name", list(SMALL))
def test_workload_reduced(name):
    """The five benchmark workloads at reduced size: forward, lse and all five gradients."""
    w = make_workload(name, **SMALL[name])
    f32 = [t.float() for t in (w.q, w.k, w.v, w.q_bias, w.k_bias)]
    o_ref, lse_ref = orc.attention_forward(*f32, None, w.causal, w.softmax_scale)
    d = w.to("cuda")
    q, k, v, qb, kb = (t.clone().requires_grad_(True) for t in (d.q, d.k, d.v, d.q_bias, d.k_bias))
    o = flash_bias_func(q, k, v, qb, kb, None, w.causal, w.softmax_scale)
    o.backward(d.do)
    torch.cuda.synchronize()
    check_close(f"{name}/o", o, o_ref, w.dtype)
    # The backward consumes the stored (rounded) output, as the reference's does: delta = rowsum(o * do)
    # is taken from the 16-bit o (flash_bias_triton.py:384-400).  The checker gets the same o, so the
    # comparison is about the backward arithmetic, not about how rounding of o propagates.
    g_ref = orc.attention_backward(w.do.float(), f32[0], f32[1], f32[2], o.detach().float().cpu(), lse_ref,
                                   f32[3], f32[4], None, w.causal, w.softmax_scale)
    for key, t, ref in zip(GRADS, (q, k, v, qb, kb), g_ref):
        check_close(f"{name}/{key}", t.grad, ref, w.dtype)


def test_tensor_path_is_selected_for_benchmark_shapes():
    import ctypes as C
    from flashbias_b200.flash_bias import _fill_common, _strides_bhs
    w = make_workload("alibi", B=1, H=2, S=256, D=32).to("cuda")
    p = _lib.FbParams()
    _fill_common(p, w.q, w.k, w.v, w.q_bias, w.k_bias, None, True, w.softmax_scale, 0)
    o = torch.empty_like(w.q)
    lse = torch.empty(1, 2, 256, device="cuda")
    p.o, p.o_stride, p.lse, p.lse_stride_bh = o.data_ptr(), _strides_bhs(o), lse.data_ptr(), 256
    assert _lib.load().fb_fwd_uses_tensor_path(C.byref(p)) == 1


def test_matches_reference_operator_semantics_default_scale_and_no_bias():
    g = torch.Generator().manual_seed(7)
    q, k, v = (torch.randn(1, 130, 2, 64, generator=g).half().cuda() for _ in range(3))
    o = flash_bias_func(q, k, v)  # no bias, default scale 1/sqrt(d), non-causal
    o_ref, _ = orc.attention_forward(q.cpu().float(), k.cpu().float(), v.cpu().float())
    check_close("nobias/o", o, o_ref, torch.float16)


# Every tensor-core kernel variant (head_dim x packed rank x scale kind), ragged and causal shapes, broadcast
# patterns of the factors: (B, H, Sq, Sk, D, R, causal, scale (None = 1/sqrt(D)), factor batch bcast, head bcast,
# dtype, backward on the tensor path)
VARIANTS = [
    (2, 3, 384, 384, 32, 0, False, None, False, False, torch.bfloat16, True),
    (1, 2, 300, 300, 32, 0, True, 0.25, False, False, torch.float16, True),     # power-of-two scale, ragged
    (2, 2, 256, 384, 32, 8, False, 0.25, True, False, torch.bfloat16, True),    # factors shared over batch
    (1, 4, 384, 256, 32, 12, True, None, False, True, torch.float16, True),     # causal Sq > Sk, shared over heads
    (1, 2, 256, 256, 32, 24, False, None, True, True, torch.bfloat16, True),    # packed rank 64
    (1, 2, 130, 400, 32, 4, True, None, False, False, torch.bfloat16, True),    # causal Sq < Sk: key tiles no query sees
    (1, 2, 384, 384, 64, 0, True, None, False, False, torch.bfloat16, True),
    (2, 2, 256, 256, 64, 12, False, None, False, True, torch.bfloat16, True),   # head_dim 64, packed rank 32
    (2, 2, 256, 256, 64, 12, False, None, False, True, torch.float16, False),   # fp16 + power-of-two scale: split form,
                                                                                 # which does not fit the backward here
    (1, 2, 200, 456, 64, 5, False, 0.1, True, False, torch.bfloat16, True),     # scale not a power of two
    (1, 2, 256, 256, 128, 8, False, None, False, False, torch.bfloat16, False),  # backward: shape-generic
    (1, 2, 256, 256, 32, 40, False, None, False, False, torch.bfloat16, False),  # rank too large for the backward
    (1, 2, 256, 256, 128, 40, False, None, False, False, torch.bfloat16, False),  # head_dim 128, packed rank 64, split scale
    (1, 2, 256, 256, 64, 40, False, 0.125, False, False, torch.float16, False),   # head_dim 64, packed rank 64
    (1, 2, 200, 200, 64, 70, False, None, False, False, torch.bfloat16, False),   # packed rank 128
]


@pytest.mark.parametrize("case", VARIANTS, ids=lambda c: "B%dH%dSq%dSk%dD%dR%d%s" % (c[0], c[1], c[2], c[3], c[4], c[5],
                                                                                  "c" if c[6] else ""))
def test_tensor_kernel_variants(case):
    import ctypes as C
    from flashbias_b200.flash_bias import _fill_common
    B, H, Sq, Sk, D, R, causal, scale, bb, hb, dtype, bwd_tensor = case
    g = torch.Generator().manual_seed(1234 + Sq + 7 * D + R)
    q, do = (torch.randn(B, Sq, H, D, generator=g) for _ in range(2))
    k, v = (torch.randn(B, Sk, H, D, generator=g) for _ in range(2))
    qb = kb = None
    if R:
        qb = torch.randn(1 if bb else B, Sq, 1 if hb else H, R, generator=g) * 0.5
        kb = torch.randn(1 if bb else B, Sk, 1 if hb else H, R, generator=g) * 0.5
    host = [t.to(dtype) if t is not None else None for t in (q, k, v, qb, kb, do)]
    dev = [t.cuda() if t is not None else None for t in host]
    p = _lib.FbParams()
    _fill_common(p, dev[0], dev[1], dev[2], dev[3], dev[4], None, causal, float(scale or 1.0 / math.sqrt(D)), 0)
    o_buf = torch.empty_like(dev[0])
    lse_buf = torch.empty(B, H, math.ceil(Sq / 128) * 128, device="cuda")
    p.o, p.o_stride = o_buf.data_ptr(), _lib.I64x3(o_buf.stride(0), o_buf.stride(2), o_buf.stride(1))
    p.lse, p.lse_stride_bh = lse_buf.data_ptr(), lse_buf.shape[-1]
    assert _lib.load().fb_fwd_uses_tensor_path(C.byref(p)) == (1 if R <= 128 else 0)
    assert _lib.load().fb_bwd_uses_tensor_path(C.byref(p)) == (1 if bwd_tensor else 0)

    leaves = [t.clone().requires_grad_(True) if t is not None else None for t in dev[:5]]
    o = flash_bias_func(leaves[0], leaves[1], leaves[2], leaves[3], leaves[4], None, causal, scale)
    o.backward(dev[5])
    torch.cuda.synchronize()
    f32 = [t.float() if t is not None else None for t in host]
    o_ref, lse_ref = orc.attention_forward(f32[0], f32[1], f32[2], f32[3], f32[4], None, causal, scale)
    tag = "variant/B%dH%dSq%dSk%dD%dR%d%s/%s" % (B, H, Sq, Sk, D, R, "c" if causal else "", str(dtype)[6:])
    check_close(f"{tag}/o", o, o_ref, dtype)
    g_ref = orc.attention_backward(f32[5], f32[0], f32[1], f32[2], o.detach().float().cpu(), lse_ref, f32[3], f32[4],
                                   None, causal, scale)
    for key, t, ref in zip(GRADS, leaves, g_ref):
        if t is not None:
            check_close(f"{tag}/{key}", t.grad, ref, dtype)
