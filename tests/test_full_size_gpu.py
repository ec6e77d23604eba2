"""The five benchmark workloads at their full benchmark sizes.

The CUDA path runs the whole problem; the CPU checker re-computes a subset of (batch, head) slices
(each slice is an independent attention problem, so a slice of the full result must match the checker
run on the sliced inputs) with the same tolerances as the reduced-size tests.  Factor gradients are
checked where the factor is not broadcast over the dimension that was subsampled."""
import pytest
import torch

from flashbias_b200 import flash_bias_func
from flashbias_b200.workloads import make_workload, swin_shift_mask
from oracle import flashbias_oracle as orc
from tests.helpers import check_close

pytestmark = pytest.mark.gpu

# workload -> (sizes, [(batch, head), ...] slices to verify)
CASES = {
    "generic": (dict(B=2, H=4, S=1024, D=32, R=8), [(b, h) for b in range(2) for h in range(4)]),
    "alibi": (dict(B=1, H=50, S=8192, D=32), [(0, 0), (0, 24), (0, 49)]),
    "swin": (dict(B=4096, H=24, window=16, D=32, R=16), [(0, 0), (2047, 11), (4095, 23)]),
    "pde": (dict(B=2, H=8, S=32768, D=64), [(1, 7)]),
    "pairformer": (dict(B=1, H=16, S=1536, D=32, R=32), [(0, 0), (0, 15)]),
}


def _slice(t, b, h):
    bb = 0 if t.shape[0] == 1 else b
    hh = 0 if t.shape[2] == 1 else h
    return t[bb:bb + 1, :, hh:hh + 1].float().contiguous()


@pytest.mark.parametrize("name", list(CASES))
def test_full_size_slices_match_checker(name):
    sizes, slices = CASES[name]
    w = make_workload(name, **sizes)
    d = w.to("cuda")
    q, k, v, qb, kb = (t.requires_grad_(True) for t in (d.q, d.k, d.v, d.q_bias, d.k_bias))
    o = flash_bias_func(q, k, v, qb, kb, None, w.causal, w.softmax_scale)
    o.backward(d.do)
    torch.cuda.synchronize()
    assert torch.isfinite(o).all()
    B, H = w.q.shape[0], w.q.shape[2]
    # factor gradients can be compared on a slice only if the factor has its own row for that (b, h)
    qb_own = (w.q_bias.shape[0] == B or B == 1) and (w.q_bias.shape[2] == H or H == 1)
    kb_own = (w.k_bias.shape[0] == B or B == 1) and (w.k_bias.shape[2] == H or H == 1)
    for (b, h) in slices:
        ins = [_slice(t, b, h) for t in (w.q, w.k, w.v, w.q_bias, w.k_bias)]
        o_ref, lse_ref = orc.attention_forward(*ins, None, w.causal, w.softmax_scale)
        o_got = o[b:b + 1, :, h:h + 1].detach().float().cpu()
        check_close(f"{name}[{b},{h}]/o", o_got, o_ref, w.dtype)
        g_ref = orc.attention_backward(_slice(w.do, b, h), ins[0], ins[1], ins[2], o_got, lse_ref, ins[3], ins[4],
                                       None, w.causal, w.softmax_scale)
        for key, t, ref in zip(("dq", "dk", "dv"), (q, k, v), g_ref[:3]):
            check_close(f"{name}[{b},{h}]/{key}", t.grad[b:b + 1, :, h:h + 1], ref, w.dtype)
        g64 = None
        for key, own, t, idx in (("dq_bias", qb_own, qb, 3), ("dk_bias", kb_own, kb, 4)):
            if not own:
                continue
            bb, hh = (0 if t.shape[0] == 1 else b), (0 if t.shape[2] == 1 else h)
            got = t.grad[bb:bb + 1, :, hh:hh + 1]
            try:
                check_close(f"{name}[{b},{h}]/{key}", got, g_ref[idx], w.dtype)
            except AssertionError:
                # Conditioning: with ALiBi-sized factors (|k_bias| up to ~7400) the fp32 logits themselves carry
                # ~4e-4 of rounding noise, which dq_bias = dS.k_bias amplifies by the factor magnitude, so an
                # fp32 evaluation -- the checker's included -- is only accurate to a few units here.  Judge
                # against an fp64 evaluation instead: the kernel must be as accurate as the fp32 checker is,
                # up to a small factor, on top of the usual 16-bit bound.
                if g64 is None:
                    o64, lse64 = orc.attention_forward(*ins, None, w.causal, w.softmax_scale, dtype=torch.float64)
                    g64 = orc.attention_backward(_slice(w.do, b, h), ins[0], ins[1], ins[2], o_got, lse64, ins[3],
                                                 ins[4], None, w.causal, w.softmax_scale, dtype=torch.float64)
                truth = g64[idx]
                err_kernel = (got.detach().double().cpu() - truth).abs().max().item()
                err_fp32 = (g_ref[idx].double() - truth).abs().max().item()
                bound = 4.0 * err_fp32 + 2e-2 * max(1.0, truth.abs().max().item())
                assert err_kernel <= bound, f"{name}[{b},{h}]/{key}: {err_kernel:.3e} > {bound:.3e} (fp32 checker {err_fp32:.3e})"


def test_full_size_swin_with_shift_mask():
    """The windowed workload at full size with the shifted-window mask (64 mask entries read as b % 64, never
    expanded to the 4096 windows): slices with and without masked regions against the checker."""
    sizes = dict(B=4096, H=24, window=16, D=32, R=16)
    w = make_workload("swin", **sizes)
    mask = swin_shift_mask(16, 8)
    d = w.to("cuda")
    q, k, v, qb, kb = (t.requires_grad_(True) for t in (d.q, d.k, d.v, d.q_bias, d.k_bias))
    o = flash_bias_func(q, k, v, qb, kb, mask.cuda(), False, w.softmax_scale)
    o.backward(d.do)
    torch.cuda.synchronize()
    assert torch.isfinite(o).all()
    for (b, h) in [(0, 0), (63, 5), (4039, 17), (4095, 23)]:   # windows 0 (no regions), 63, 7 (two regions), 63 (four)
        ins = [_slice(t, b, h) for t in (w.q, w.k, w.v, w.q_bias, w.k_bias)]
        m = mask[b % 64:b % 64 + 1]
        o_ref, lse_ref = orc.attention_forward(*ins, m, False, w.softmax_scale)
        o_got = o[b:b + 1, :, h:h + 1].detach().float().cpu()
        check_close(f"swin_shifted[{b},{h}]/o", o_got, o_ref, w.dtype)
        g_ref = orc.attention_backward(_slice(w.do, b, h), ins[0], ins[1], ins[2], o_got, lse_ref, ins[3], ins[4], m,
                                       False, w.softmax_scale)
        for key, t, ref in zip(("dq", "dk", "dv"), (q, k, v), g_ref[:3]):
            check_close(f"swin_shifted[{b},{h}]/{key}", t.grad[b:b + 1, :, h:h + 1], ref, w.dtype)


def test_full_size_softmax_rows_sum_to_one():
    """Size-independent property at the largest sequence length: with v = 1 the output is exactly the row
    sum of the probabilities, i.e. 1 for every row."""
    w = make_workload("pde", B=1, H=2, S=32768, D=64).to("cuda")
    o = flash_bias_func(w.q, w.k, torch.ones_like(w.v), w.q_bias, w.k_bias, None, False, w.softmax_scale)
    torch.cuda.synchronize()
    assert (o.float() - 1.0).abs().max().item() < 1e-2
