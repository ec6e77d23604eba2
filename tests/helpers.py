"""Shared helpers for the parity tests: golden loading and tolerance checks."""
import glob
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
DTYPES = {"torch.float16": torch.float16, "torch.bfloat16": torch.bfloat16, "torch.float32": torch.float32}

# Tolerances of the parity contract for fp16/bf16 outputs and gradients:
# max-abs against the fp32 checker, and relative L2 against the fp32 checker
# rounded to the output dtype.
MAX_ABS_TOL = 2e-2
REL_L2_TOL = 1e-3


# Achieved errors of every check_close call of the session, keyed by the check's name: dumped as JSON to the path
# in the environment variable FB_PARITY_REPORT (if set) when the session ends (tests/conftest.py).
ACHIEVED = {}


def golden_names():
    return sorted(os.path.splitext(os.path.basename(p))[0] for p in glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))


def load_golden(name):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    B, Sq, Sk, H, D, R, causal = (int(x) for x in z["meta"])
    case = dict(name=name, B=B, Sq=Sq, Sk=Sk, H=H, D=D, R=R, causal=bool(causal),
                scale=float(z["scale"][0]), dtype=DTYPES[str(z["dtype"][0])])
    ins = {k[3:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("in_")}
    outs = {k: torch.from_numpy(z[k]) for k in ("o", "dq", "dk", "dv", "dq_bias", "dk_bias") if k in z.files}
    return case, ins, outs


def rel_l2(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def max_abs(a, b):
    return float((a.double() - b.double()).abs().max())


def check_close(name, got, want_fp32, out_dtype, max_abs_tol=MAX_ABS_TOL, rel_l2_tol=REL_L2_TOL):
    """Gate `got` (any dtype) against the fp32 checker value.

    (i) max-abs <= 2e-2 * max(1, max|want|) against the raw fp32 value.  The bound is absolute for
        values of order one and scales with the largest magnitude beyond that: half a bf16 ulp of a
        value near 4.7 is already 1.6e-2, so an unscaled bound cannot hold for large gradients.
    (ii) relative L2 against the fp32 value rounded to the output dtype: <= 1e-3 for fp16 outputs,
        <= 4e-3 for bf16 outputs (8 mantissa bits in P, dS and the stored result).
    """
    got = got.detach().float().cpu()
    want = want_fp32.detach().float().cpu()
    assert got.shape == want.shape, f"{name}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{name}: non-finite values"
    mag = float(want.abs().max())
    tol = max_abs_tol * max(1.0, mag)
    ma = max_abs(got, want)
    rl = rel_l2(got, want.to(out_dtype).float())
    ACHIEVED[name] = {"max_abs": ma, "rel_l2_vs_rounded": rl, "rel_l2_vs_fp32": rel_l2(got, want), "want_max": mag,
                      "dtype": str(out_dtype).replace("torch.", "")}
    assert ma <= tol, f"{name}: max-abs {ma:.3e} > {tol:.3e} (|want|max {mag:.3e}, rel-l2 {rl:.3e})"
    gate = rel_l2_tol * (4.0 if out_dtype == torch.bfloat16 else 1.0)
    assert rl <= gate, f"{name}: rel-l2 {rl:.3e} > {gate:.1e} (max-abs {ma:.3e})"
    return ma, rl
