"""Second oracle: the reference's own Triton kernel (flash_bias/flash_bias_triton.py), run on the same GPU on
the same seeded inputs.  The unmodified file is expected under baseline/_ref/ (it is not part of this
repository); without it, or if Triton cannot compile it for this GPU, the test records why and skips.  The
product never calls it.

The Triton kernel is itself an approximation (its bias dot runs in TF32 and its backward has known races on
newer Triton releases, flash_bias/README.md:12), so the gate is triangular: this library must be at least as
close to the fp32 checker as the parity contract demands, and its distance to the Triton result may not
exceed the Triton kernel's own distance to the checker plus that tolerance."""
import os
import sys

import pytest
import torch

from flashbias_b200 import flash_bias_func
from flashbias_b200.workloads import make_workload
from oracle import flashbias_oracle as orc
from tests.helpers import ACHIEVED, check_close, max_abs

pytestmark = pytest.mark.gpu

REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")

CASES = {
    "generic": dict(B=2, H=4, S=1024, D=32, R=8),      # the reference's own benchmark shape, full size
    "alibi": dict(B=1, H=4, S=1024, D=32),             # reduced causal ALiBi
    "pairformer": dict(B=1, H=4, S=512, D=32, R=32),   # reduced pair-bias
}


def _triton_func():
    if not os.path.exists(os.path.join(REF_DIR, "flash_bias_triton.py")):
        pytest.skip("baseline/_ref/flash_bias_triton.py is not present")
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    try:
        import flash_bias_triton
    except Exception as e:  # pragma: no cover
        pytest.skip(f"reference Triton kernel failed to import: {type(e).__name__}: {e}")
    return flash_bias_triton.flash_bias_func


@pytest.mark.parametrize("name", list(CASES))
def test_against_reference_triton_kernel(name):
    ref_func = _triton_func()
    w = make_workload(name, **CASES[name])
    d = w.to("cuda")
    sh = w.shape
    f32 = [t.float() for t in (w.q, w.k, w.v, w.q_bias, w.k_bias)]
    o_ref, lse_ref = orc.attention_forward(*f32, None, w.causal, w.softmax_scale)

    ours = [t.clone().requires_grad_(True) for t in (d.q, d.k, d.v, d.q_bias, d.k_bias)]
    o = flash_bias_func(*ours, None, w.causal, w.softmax_scale)
    o.backward(d.do)
    torch.cuda.synchronize()
    check_close(f"triton2nd/{name}/ours/o", o, o_ref, w.dtype)

    # the reference's backward indexes factors with un-expanded strides: give it expanded, contiguous factors
    theirs = [t.clone().requires_grad_(True) for t in (d.q, d.k, d.v)]
    qb_t = d.q_bias.expand(sh["B"], -1, sh["H"], -1).contiguous().requires_grad_(True)
    kb_t = d.k_bias.expand(sh["B"], -1, sh["H"], -1).contiguous().requires_grad_(True)
    try:
        o_t = ref_func(theirs[0], theirs[1], theirs[2], qb_t, kb_t, None, w.causal, w.softmax_scale)
        o_t.backward(d.do)
        torch.cuda.synchronize()
    except Exception as e:
        ACHIEVED[f"triton2nd/{name}/triton"] = {"failed": f"{type(e).__name__}: {str(e)[:300]}"}
        pytest.skip(f"reference Triton kernel did not run here: {type(e).__name__}: {str(e)[:200]}")
    d_triton = max_abs(o_t.float().cpu(), o_ref)
    d_ours = max_abs(o.float().cpu(), o_ref)
    d_between = max_abs(o.float().cpu(), o_t.float().cpu())
    rec = {"o": {"triton_vs_checker": d_triton, "ours_vs_checker": d_ours, "ours_vs_triton": d_between}}
    assert d_between <= d_triton + 2e-2, f"{name}: ours vs Triton {d_between:.3e}, Triton vs checker {d_triton:.3e}"
    g_ref = orc.attention_backward(w.do.float(), f32[0], f32[1], f32[2], o.detach().float().cpu(), lse_ref,
                                   f32[3], f32[4], None, w.causal, w.softmax_scale)
    for key, mine, his, want in zip(("dq", "dk", "dv"), ours[:3], theirs, g_ref[:3]):
        dt, do_, db = (max_abs(his.grad.float().cpu(), want), max_abs(mine.grad.float().cpu(), want),
                       max_abs(mine.grad.float().cpu(), his.grad.float().cpu()))
        rec[key] = {"triton_vs_checker": dt, "ours_vs_checker": do_, "ours_vs_triton": db}
        tol = 2e-2 * max(1.0, float(want.abs().max()))
        assert do_ <= tol, f"{name}/{key}: ours vs checker {do_:.3e} > {tol:.3e}"
        assert db <= dt + tol, f"{name}/{key}: ours vs Triton {db:.3e}, Triton vs checker {dt:.3e}"
    ACHIEVED[f"triton2nd/{name}"] = rec
    print(f"\n[triton second oracle] {name}: {rec}")
