"""Parity of the paths beside the plain factor form: additive masks on the tensor-core kernels, the fused
ALiBi producer, rank 96, factors shared by many (batch, head) pairs, expanded-view factors, permuted
(B, H, S, D) inputs, and the device status word.  All through the C ABI / the public operators, against
the CPU checker."""
import ctypes as C
import math

import pytest
import torch

from flashbias_b200 import _lib, check_device_status, flash_bias_alibi_func, flash_bias_func
from flashbias_b200.flash_bias import _fill_common, _strides_bhs, flash_bias_backward, flash_bias_forward
from flashbias_b200.workloads import make_workload
from oracle import flashbias_oracle as orc
from tests.helpers import check_close, load_golden

pytestmark = pytest.mark.gpu

GRADS = ("dq", "dk", "dv", "dq_bias", "dk_bias")


def _uses_tensor_path(q, k, v, qb, kb, mask, causal, scale, slopes=None):
    p = _lib.FbParams()
    _fill_common(p, q, k, v, qb, kb, mask, causal, float(scale), 0, slopes)
    o = torch.empty_like(q)
    lse = torch.empty(q.shape[0], q.shape[2], math.ceil(q.shape[1] / 128) * 128, device=q.device)
    p.o, p.o_stride, p.lse, p.lse_stride_bh = o.data_ptr(), _strides_bhs(o), lse.data_ptr(), lse.shape[-1]
    lib = _lib.load()
    return lib.fb_fwd_uses_tensor_path(C.byref(p)), lib.fb_bwd_uses_tensor_path(C.byref(p))


def _expand_mask(mask, B):
    """The checker's view of a periodic mask: entry b reads mask[b % n]."""
    if mask is None or mask.shape[0] in (1, B):
        return mask
    return mask.repeat(B // mask.shape[0], 1, 1, 1)


def _check_all(tag, host, mask, causal, scale, dtype, flags=0):
    """Forward + backward of the operator on `host` = (q, k, v, q_bias, k_bias, do) (already rounded to dtype)
    against the checker on the same values."""
    dev = [t.cuda() if t is not None else None for t in host]
    mdev = mask.cuda() if mask is not None else None
    o, lse, sc = flash_bias_forward(dev[0], dev[1], dev[2], dev[3], dev[4], mdev, causal, scale, flags=flags)
    grads = flash_bias_backward(dev[5], dev[0], dev[1], dev[2], o, dev[3], dev[4], lse, mdev, causal, sc, flags=flags)
    torch.cuda.synchronize()
    check_device_status()
    f32 = [t.float() if t is not None else None for t in host]
    m32 = _expand_mask(mask, host[0].shape[0])
    m32 = m32.float() if m32 is not None else None
    o_ref, lse_ref = orc.attention_forward(f32[0], f32[1], f32[2], f32[3], f32[4], m32, causal, scale)
    check_close(f"{tag}/o", o, o_ref, dtype)
    Sq = host[0].shape[1]
    finite = torch.isfinite(lse_ref)
    assert (lse[:, :, :Sq].float().cpu()[finite] - lse_ref[finite]).abs().max().item() < 2e-2
    g_ref = orc.attention_backward(f32[5], f32[0], f32[1], f32[2], o.float().cpu(), lse_ref, f32[3], f32[4], m32,
                                   causal, scale)
    for key, g, want in zip(GRADS, grads, g_ref):
        if want is not None:
            check_close(f"{tag}/{key}", g, want, dtype)


# ---------------------------------------------------------------------------------------------------------------
# additive masks on the tensor-core kernels
# ---------------------------------------------------------------------------------------------------------------
# (B, H, Sq, Sk, D, R, causal, mask batch entries, mask heads, mask rows (1 = vector), mask dtype, dtype)
MASK_CASES = [
    (2, 2, 256, 256, 32, 8, False, 2, 1, 256, torch.float32, torch.bfloat16),     # Swin-like: per-window matrix, fp32
    (8, 3, 256, 256, 32, 16, False, 4, 1, 256, torch.float32, torch.float16),     # periodic batch: b % 4
    (2, 2, 200, 330, 32, 4, False, 2, 1, 1, torch.float32, torch.float16),        # key-padding vector, ragged
    (1, 2, 300, 300, 64, 0, True, 1, 2, 300, torch.bfloat16, torch.bfloat16),     # dense bias through the mask, 16-bit
    (2, 2, 130, 257, 64, 5, False, 1, 1, 130, torch.float16, torch.float16),      # unaligned rows: scalar loads
    (1, 2, 256, 384, 128, 0, False, 1, 2, 256, torch.float32, torch.bfloat16),    # head_dim 128 (forward tensor path)
]


@pytest.mark.parametrize("case", MASK_CASES, ids=lambda c: "B%dH%dSq%dSk%dD%dR%dm%dx%dx%d" % (c[0], c[1], c[2], c[3], c[4], c[5], c[7], c[8], c[9]))
def test_masks_on_tensor_path(case):
    B, H, Sq, Sk, D, R, causal, mB, mH, mRows, mdtype, dtype = case
    g = torch.Generator().manual_seed(99 + Sq + D + R)
    q, do = (torch.randn(B, Sq, H, D, generator=g) for _ in range(2))
    k, v = (torch.randn(B, Sk, H, D, generator=g) for _ in range(2))
    qb = kb = None
    if R:
        qb = torch.randn(1, Sq, H, R, generator=g) * 0.5
        kb = torch.randn(1, Sk, H, R, generator=g) * 0.5
    mask = torch.randn(mB, mH, mRows, Sk, generator=g)
    # blocks of masked-out entries as a shifted-window mask has them (-100), and some -inf
    mask = torch.where(torch.rand(mB, mH, mRows, Sk, generator=g) < 0.3, torch.full_like(mask, -100.0), mask)
    if mRows == 1:
        mask[..., -7:] = float("-inf")
    mask = mask.to(mdtype)
    host = [t.to(dtype) if t is not None else None for t in (q, k, v, qb, kb, do)]
    scale = 1.0 if D == 32 else None
    scale = scale or 1.0 / math.sqrt(D)
    dev = [t.cuda() if t is not None else None for t in host]
    fwd_t, bwd_t = _uses_tensor_path(dev[0], dev[1], dev[2], dev[3], dev[4], mask.cuda(), causal, scale)
    assert fwd_t == 1
    assert bwd_t == (1 if D <= 64 else 0)
    _check_all("mask/B%dH%dSq%dSk%dD%dR%d" % (B, H, Sq, Sk, D, R), host, mask, causal, scale, dtype)


@pytest.mark.parametrize("name", ["mask_vector", "mask_matrix"])
def test_mask_goldens_padded_to_head_dim_32(name):
    """The reference-generated mask goldens, with q/k/v zero-padded to head_dim 32 (and the scale kept): zero
    columns change nothing in q.k or in the first D columns of the output, so the golden values still apply and
    the case now runs on the tensor-core kernels."""
    case, ins, ref = load_golden(name)
    dtype, D = case["dtype"], case["D"]
    pad = lambda t: torch.nn.functional.pad(t, (0, 32 - D))
    host = {k: (pad(v) if k in ("q", "k", "v", "do") else v) for k, v in ins.items()}
    t = {k: v.to(dtype).cuda() for k, v in host.items() if k != "mask"}
    mask = host["mask"].cuda()
    fwd_t, bwd_t = _uses_tensor_path(t["q"], t["k"], t["v"], t["q_bias"], t["k_bias"], mask, case["causal"], case["scale"])
    assert (fwd_t, bwd_t) == (1, 1)
    o, lse, sc = flash_bias_forward(t["q"], t["k"], t["v"], t["q_bias"], t["k_bias"], mask, case["causal"], case["scale"])
    grads = flash_bias_backward(t["do"], t["q"], t["k"], t["v"], o, t["q_bias"], t["k_bias"], lse, mask, case["causal"], sc)
    torch.cuda.synchronize()
    check_close(f"{name}_d32/o", o[..., :D], ref["o"], dtype)
    for key, g in zip(GRADS, grads):
        if key in ref:
            want = ref[key]
            got = g[..., :D] if key in ("dq", "dk", "dv") else g
            check_close(f"{name}_d32/{key}/golden", got, want, dtype, rel_l2_tol=2.5e-3)


# ---------------------------------------------------------------------------------------------------------------
# fused ALiBi producer
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("case", [
    (1, 6, 1024, 1024, 32, True, torch.bfloat16, 0),
    (2, 3, 384, 384, 64, True, torch.float16, 0),
    (1, 4, 300, 520, 32, False, torch.bfloat16, 0),      # non-causal, ragged cross-attention
    (1, 2, 256, 256, 128, True, torch.bfloat16, 0),      # backward on the shape-generic kernels
    (1, 2, 200, 200, 32, True, torch.float16, _lib.FB_FLAG_FORCE_GENERAL),
], ids=lambda c: "B%dH%dSq%dSk%dD%d%s%s" % (c[0], c[1], c[2], c[3], c[4], "c" if c[5] else "", "g" if c[7] else ""))
def test_alibi_producer(case):
    """slope_h * (j - i) generated in the kernels == the checker fed the exact (unrounded) rank-2 factors
    q_bias[i] = [-m i, 1], k_bias[j] = [1, m j] in fp64."""
    B, H, Sq, Sk, D, causal, dtype, flags = case
    g = torch.Generator().manual_seed(5 + Sq + D)
    q, do = (torch.randn(B, Sq, H, D, generator=g).to(dtype) for _ in range(2))
    k, v = (torch.randn(B, Sk, H, D, generator=g).to(dtype) for _ in range(2))
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=torch.float32)
    if not causal:
        slopes = slopes * 0.05  # keep the logits of far-future keys within range
    dev = [t.cuda() for t in (q, k, v, do)]
    sl = slopes.cuda()
    fwd_t, bwd_t = _uses_tensor_path(dev[0], dev[1], dev[2], None, None, None, causal, 1.0 / math.sqrt(D), sl)
    if flags == 0:
        assert fwd_t == 1 and bwd_t == (1 if D <= 64 else 0)
    if flags:
        o, lse, sc = flash_bias_forward(dev[0], dev[1], dev[2], None, None, None, causal, None, flags=flags, alibi_slopes=sl)
        dq, dk, dv, _, _ = flash_bias_backward(dev[3], dev[0], dev[1], dev[2], o, None, None, lse, None, causal, sc,
                                               flags=flags, alibi_slopes=sl)
    else:
        leaves = [t.clone().requires_grad_(True) for t in dev[:3]]
        o = flash_bias_alibi_func(leaves[0], leaves[1], leaves[2], sl, causal, None)
        o.backward(dev[3])
        dq, dk, dv = (t.grad for t in leaves)
    torch.cuda.synchronize()
    check_device_status()
    f64 = torch.float64
    m = slopes.to(f64)
    pi, pj = torch.arange(Sq, dtype=f64), torch.arange(Sk, dtype=f64)
    qb = torch.stack([-(m[None, :] * pi[:, None]), torch.ones(Sq, H, dtype=f64)], dim=-1).unsqueeze(0)
    kb = torch.stack([torch.ones(Sk, H, dtype=f64), m[None, :] * pj[:, None]], dim=-1).unsqueeze(0)
    o_ref, lse_ref = orc.attention_forward(q, k, v, qb, kb, None, causal, None, dtype=f64)
    tag = "alibi_producer/B%dH%dSq%dSk%dD%d%s%s" % (B, H, Sq, Sk, D, "c" if causal else "", "g" if flags else "")
    check_close(f"{tag}/o", o, o_ref, dtype)
    g_ref = orc.attention_backward(do, q, k, v, o.detach().cpu(), lse_ref, qb, kb, None, causal, None, dtype=f64)
    for key, got, want in zip(("dq", "dk", "dv"), (dq, dk, dv), g_ref[:3]):
        check_close(f"{tag}/{key}", got, want, dtype)


# ---------------------------------------------------------------------------------------------------------------
# rank 96 (AlphaFold3 triangle attention): forward on the tensor-core kernel
# ---------------------------------------------------------------------------------------------------------------
def test_rank_96_forward_on_tensor_path():
    B, S, H, D, R = 64, 512, 4, 32, 96
    g = torch.Generator().manual_seed(96)
    q, k, v, do = (torch.randn(B, S, H, D, generator=g) for _ in range(4))
    q = q / math.sqrt(D)  # the call site divides q by sqrt(c) and passes scale 1
    qb = torch.tanh(torch.randn(1, S, H, R, generator=g)) * 0.3
    kb = torch.tanh(torch.randn(1, S, H, R, generator=g)) * 0.3
    dtype = torch.float16
    host = [t.to(dtype) for t in (q, k, v, qb, kb, do)]
    dev = [t.cuda() for t in host]
    fwd_t, bwd_t = _uses_tensor_path(dev[0], dev[1], dev[2], dev[3], dev[4], None, False, 1.0)
    assert fwd_t == 1 and bwd_t == 0
    o, lse, _ = flash_bias_forward(dev[0], dev[1], dev[2], dev[3], dev[4], None, False, 1.0)
    torch.cuda.synchronize()
    sel = [0, 31, 63]
    f32 = [host[i][sel].float() for i in range(3)] + [host[3].float(), host[4].float()]
    o_ref, lse_ref = orc.attention_forward(*f32, None, False, 1.0)
    check_close("rank96/o", o[sel], o_ref, dtype)
    assert (lse[sel][:, :, :S].float().cpu() - lse_ref).abs().max().item() < 2e-2


def test_rank_96_small_forward_backward():
    """Rank 96 end to end (backward on the shape-generic kernels), small enough for the whole checker."""
    B, S, H, D, R = 2, 200, 2, 32, 96
    g = torch.Generator().manual_seed(97)
    q, k, v, do = (torch.randn(B, S, H, D, generator=g) for _ in range(4))
    qb = torch.tanh(torch.randn(1, S, H, R, generator=g)) * 0.3
    kb = torch.tanh(torch.randn(1, S, H, R, generator=g)) * 0.3
    host = [t.to(torch.float16) for t in (q, k, v, qb, kb, do)]
    _check_all("rank96_small", host, None, False, 1.0, torch.float16)


# ---------------------------------------------------------------------------------------------------------------
# factors shared by more (batch, head) pairs than the backward keeps accumulator copies (64)
# ---------------------------------------------------------------------------------------------------------------
def test_factor_gradients_shared_by_256_windows():
    """Swin shape: one factor pair per head shared by 256 windows; dq_bias / dk_bias are sums over the whole
    batch and are checked over the whole batch."""
    w = make_workload("swin", B=256, H=24, window=16, D=32, R=16)
    host = [w.q, w.k, w.v, w.q_bias, w.k_bias, w.do]
    _check_all("swin_shared256", host, None, w.causal, w.softmax_scale, w.dtype)


def test_factor_gradients_shared_over_heads_long_sequence():
    """PDE shape: factors shared by the 8 heads of each batch entry at a long sequence."""
    w = make_workload("pde", B=2, H=8, S=4096, D=64)
    host = [w.q, w.k, w.v, w.q_bias, w.k_bias, w.do]
    _check_all("pde_shared_heads", host, None, w.causal, w.softmax_scale, w.dtype)


def test_factors_shared_over_batch_and_heads_many_pairs():
    """One factor pair for everything: 96 (batch, head) pairs add into the same accumulator rows."""
    B, H, S, D, R = 16, 6, 256, 32, 8
    g = torch.Generator().manual_seed(4242)
    q, k, v, do = (torch.randn(B, S, H, D, generator=g) for _ in range(4))
    qb, kb = (torch.randn(1, S, 1, R, generator=g) * 0.5 for _ in range(2))
    host = [t.to(torch.bfloat16) for t in (q, k, v, qb, kb, do)]
    _check_all("shared_all96", host, None, False, None, torch.bfloat16)


# ---------------------------------------------------------------------------------------------------------------
# the two forms of the query-major backward (one work item per CTA / one persistent CTA per SM)
# ---------------------------------------------------------------------------------------------------------------
# (B, H, Sq, Sk, R, causal, scale, masked, dtype): head_dim 32 with factor operands
BWD_FORM_CASES = [
    (40, 6, 256, 256, 16, False, None, False, torch.bfloat16),    # windowed shape: 480 items of two query tiles
    (40, 6, 256, 256, 16, False, None, True, torch.bfloat16),     # ... with a shifted-window mask, period 4
    (2, 40, 1024, 1024, 2, True, None, False, torch.bfloat16),    # causal: items of 8 ... 1 query tiles
    (3, 50, 200, 1000, 8, True, 0.25, False, torch.float16),      # causal, Sq < Sk: key tiles no query sees; scale 2^-2
    (5, 31, 130, 257, 24, False, 1.0, False, torch.float16),      # ragged tiles, packed rank 32, scale 1
    (1, 3, 384, 384, 28, False, None, False, torch.bfloat16),     # fewer items than SMs, packed rank 64
    (2, 37, 640, 512, 12, True, 0.125, False, torch.bfloat16),    # causal, Sq > Sk, bf16 with a power-of-two scale
]


@pytest.mark.parametrize("case", BWD_FORM_CASES, ids=lambda c: "B%dH%dSq%dSk%dR%d%s%s" % (c[0], c[1], c[2], c[3], c[4], "c" if c[5] else "", "m" if c[7] else ""))
def test_backward_persistent_and_one_item_forms_agree(case):
    B, H, Sq, Sk, R, causal, scale, masked, dtype = case
    D = 32
    g = torch.Generator().manual_seed(1234 + Sq + R)
    q, do = (torch.randn(B, Sq, H, D, generator=g) for _ in range(2))
    k, v = (torch.randn(B, Sk, H, D, generator=g) for _ in range(2))
    qb = torch.randn(1, Sq, H, R, generator=g) * 0.5       # shared by the batch: bulk reductions from many CTAs
    kb = torch.randn(1, Sk, H, R, generator=g) * 0.5
    mask = None
    if masked:
        mask = torch.where(torch.rand(4, 1, Sq, Sk, generator=g) < 0.3, torch.tensor(-100.0), torch.tensor(0.0))
    host = [t.to(dtype) for t in (q, k, v, qb, kb, do)]
    scale = scale or 1.0 / math.sqrt(D)
    tag = "bwdform/B%dH%dSq%dSk%dR%d%s%s" % (B, H, Sq, Sk, R, "c" if causal else "", "m" if masked else "")
    out = {}
    for name, flag in (("one_item", _lib.FB_FLAG_BWD_ONE_ITEM), ("persistent", _lib.FB_FLAG_BWD_PERSISTENT)):
        _check_all(f"{tag}/{name}", host, mask, causal, scale, dtype, flags=flag)
        dev = [t.cuda() for t in host]
        mdev = mask.cuda() if mask is not None else None
        o, lse, sc = flash_bias_forward(dev[0], dev[1], dev[2], dev[3], dev[4], mdev, causal, scale, flags=flag)
        out[name] = flash_bias_backward(dev[5], dev[0], dev[1], dev[2], o, dev[3], dev[4], lse, mdev, causal, sc,
                                        flags=flag)
        torch.cuda.synchronize()
        check_device_status()
    # same arithmetic per work item in both forms: dk and dv are bit-identical; dq and the factor gradients are
    # fp32 sums whose order depends on the schedule
    assert torch.equal(out["one_item"][1], out["persistent"][1])
    assert torch.equal(out["one_item"][2], out["persistent"][2])
    for i in (0, 3, 4):
        a, b = out["one_item"][i].float(), out["persistent"][i].float()
        assert (a - b).abs().max().item() <= 2e-2 * max(1.0, a.abs().max().item())


# ---------------------------------------------------------------------------------------------------------------
# operator-level behaviour
# ---------------------------------------------------------------------------------------------------------------
def test_expanded_view_factors_get_summed_gradients():
    """A factor passed as an expanded view (stride 0, size > 1) is a broadcast factor: its .grad is the sum over
    the expanded dimension, as autograd of the naive path gives."""
    B, H, S, D, R = 3, 2, 160, 32, 8
    g = torch.Generator().manual_seed(31)
    q, k, v, do = (torch.randn(B, S, H, D, generator=g).half().cuda() for _ in range(4))
    qb0 = (torch.randn(1, S, H, R, generator=g) * 0.5).half().cuda().requires_grad_(True)
    kb0 = (torch.randn(1, S, 1, R, generator=g) * 0.5).half().cuda().requires_grad_(True)
    o = flash_bias_func(q, k, v, qb0.expand(B, -1, -1, -1), kb0.expand(B, -1, H, -1), None, False, None)
    o.backward(do)
    torch.cuda.synchronize()
    f = lambda t: t.detach().float().cpu()
    o_ref, lse_ref = orc.attention_forward(f(q), f(k), f(v), f(qb0), f(kb0))
    g_ref = orc.attention_backward(f(do), f(q), f(k), f(v), f(o), lse_ref, f(qb0), f(kb0))
    check_close("expanded/o", o, o_ref, torch.float16)
    check_close("expanded/dq_bias", qb0.grad, g_ref[3], torch.float16)
    check_close("expanded/dk_bias", kb0.grad, g_ref[4], torch.float16)


def test_permuted_bhsd_inputs_run_on_the_tensor_path_without_copies():
    """Call sites hold (B, H, S, D) tensors and permute them; the permuted views (no .contiguous()) are taken as
    they are: the C ABI addresses (batch, head, row) through strides."""
    B, H, S, D, R = 2, 4, 256, 32, 16
    g = torch.Generator().manual_seed(77)
    qh, kh, vh = (torch.randn(B, H, S, D, generator=g).half().cuda() for _ in range(3))
    qbh, kbh = ((torch.randn(1, H, S, R, generator=g) * 0.5).half().cuda() for _ in range(2))
    q, k, v, qb, kb = (t.permute(0, 2, 1, 3) for t in (qh, kh, vh, qbh, kbh))
    assert not q.is_contiguous()
    fwd_t, bwd_t = _uses_tensor_path(q, k, v, qb, kb, None, False, 1.0)
    assert (fwd_t, bwd_t) == (1, 1)
    o = flash_bias_func(q, k, v, qb, kb, None, False, 1.0)
    o2 = flash_bias_func(*(t.contiguous() for t in (q, k, v, qb, kb)), None, False, 1.0)
    torch.cuda.synchronize()
    assert torch.equal(o, o2)


def test_status_word_round_trip():
    """fb_read_status returns FB_EDEVICE for a non-zero word and the word itself; nothing on the GPU is made to
    fail for this: the word is written by the host."""
    lib = _lib.load()
    word = torch.zeros(1, dtype=torch.int32, device="cuda")
    val = C.c_int32(-1)
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.fb_read_status(word.data_ptr(), C.byref(val), stream) == 0 and val.value == 0
    word.fill_(1)
    assert lib.fb_read_status(word.data_ptr(), C.byref(val), stream) == -10 and val.value == 1
    assert b"wait" in lib.fb_status_string(1)
    check_device_status()  # nothing has been reported by the kernels of this session


def test_fp16_power_of_two_scale_large_factors_do_not_overflow():
    """fp16 factors above 8188 with a power-of-two scale below one (head_dim 64: 1/8): dividing the q-side
    factor by the scale would leave the fp16 range, so that form is not used for fp16; the result stays finite
    and correct.  The two large columns cancel to a bias of 8 * ((j mod 4) - (i mod 4))."""
    B, H, S, D = 1, 2, 256, 64
    g = torch.Generator().manual_seed(8)
    q, k, v, do = (torch.randn(B, S, H, D, generator=g).half() for _ in range(4))
    do = (do.float() * 0.01).half()  # keeps dk_bias = dS^T.q_bias (|q_bias| ~ 8192) inside the fp16 range
    pos = torch.arange(S, dtype=torch.float32)
    big = 8192.0 + 8.0 * (pos % 4)
    qb = torch.stack([-big, torch.ones(S)], dim=-1)[None, :, None, :].expand(1, S, H, 2).contiguous().half()
    kb = torch.stack([torch.ones(S), big], dim=-1)[None, :, None, :].expand(1, S, H, 2).contiguous().half()
    assert qb.abs().max() * 8 > 65504  # pre-dividing by the scale would overflow
    dev = [t.cuda() for t in (q, k, v, qb, kb, do)]
    o, lse, sc = flash_bias_forward(dev[0], dev[1], dev[2], dev[3], dev[4], None, True, None)
    grads = flash_bias_backward(dev[5], dev[0], dev[1], dev[2], o, dev[3], dev[4], lse, None, True, sc)
    torch.cuda.synchronize()
    check_device_status()
    f32 = [t.float() for t in (q, k, v, qb, kb, do)]
    o_ref, lse_ref = orc.attention_forward(*f32[:5], None, True, None)
    check_close("fp16_pow2_large/o", o, o_ref, torch.float16)
    g_ref = orc.attention_backward(f32[5], f32[0], f32[1], f32[2], o.float().cpu(), lse_ref, f32[3], f32[4], None, True)
    for key, g, want in zip(GRADS[:3], grads[:3], g_ref[:3]):
        check_close(f"fp16_pow2_large/{key}", g, want, torch.float16)
    # factor gradients against factors of magnitude 8192: the 16-bit rounding of dS is amplified by that
    # magnitude, so only a loose relative bound applies here (the point of the case is the range, not this)
    for key, g, want in zip(GRADS[3:], grads[3:], g_ref[3:]):
        check_close(f"fp16_pow2_large/{key}", g, want, torch.float16, rel_l2_tol=2e-2)


def test_prepare_bhsd_matches_the_call_site_glue():
    """The fused cast / normalise / per-head scale against the torch ops of the Swin-V2 call site, and the
    operator on its strided result against the operator on the permuted, contiguous copy."""
    from flashbias_b200.layout import prepare_bhsd
    B, H, S, D = 4, 3, 256, 32
    g = torch.Generator().manual_seed(55)
    qkv = torch.randn(3, B, H, S, D, generator=g).cuda()  # fp32, (B, H, S, D) slices of one buffer
    logit_scale = (torch.rand(H, generator=g) * 2 + 1).cuda()
    q = prepare_bhsd(qkv[0], torch.float16, normalize=True, head_scale=logit_scale)
    k = prepare_bhsd(qkv[1], torch.float16, normalize=True)
    v = prepare_bhsd(qkv[2], torch.float16)
    q_ref = (torch.nn.functional.normalize(qkv[0], dim=-1) * logit_scale[None, :, None, None]).half().permute(0, 2, 1, 3)
    k_ref = torch.nn.functional.normalize(qkv[1], dim=-1).half().permute(0, 2, 1, 3)
    v_ref = qkv[2].half().permute(0, 2, 1, 3)
    assert q.shape == (B, S, H, D) and not q.is_contiguous()
    for got, want in ((q, q_ref), (k, k_ref), (v, v_ref)):
        assert (got.float() - want.float()).abs().max().item() <= 2e-3  # one fp16 ulp of values up to ~3
    assert torch.equal(v, v_ref)
    o = flash_bias_func(q, k, v, None, None, None, False, 1.0)
    o_ref = flash_bias_func(q.contiguous(), k.contiguous(), v.contiguous(), None, None, None, False, 1.0)
    torch.cuda.synchronize()
    assert torch.equal(o, o_ref)
    # bf16 output from a bf16 strided input
    xb = torch.randn(B, S, H, 64, generator=g).bfloat16().cuda().permute(0, 2, 1, 3)  # (B, H, S, D) view
    yb = prepare_bhsd(xb, torch.bfloat16, normalize=True)
    want = torch.nn.functional.normalize(xb.float(), dim=-1).bfloat16().permute(0, 2, 1, 3)
    assert (yb.float() - want.float()).abs().max().item() <= 8e-3
