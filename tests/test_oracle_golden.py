"""The CPU checker against golden vectors produced by the reference's own naive attention."""
import pytest
import torch

from oracle import flashbias_oracle as orc
from tests.helpers import golden_names, load_golden, max_abs


@pytest.mark.parametrize("name", golden_names())
def test_oracle_matches_reference_golden(name):
    case, ins, ref = load_golden(name)
    o, lse, (dq, dk, dv, dqb, dkb) = orc.attention_forward_backward(
        ins["q"], ins["k"], ins["v"], ins.get("q_bias"), ins.get("k_bias"), ins.get("mask"),
        case["causal"], case["scale"], ins["do"])
    got = dict(o=o, dq=dq, dk=dk, dv=dv, dq_bias=dqb, dk_bias=dkb)
    for key, want in ref.items():
        err = max_abs(got[key], want)
        scale = max(1.0, float(want.abs().max()))
        assert err <= 2e-5 * scale, f"{name}/{key}: {err}"


def test_oracle_fp64_agrees_with_fp32():
    case, ins, ref = load_golden("c1_small")
    o64, _, g64 = orc.attention_forward_backward(
        ins["q"], ins["k"], ins["v"], ins["q_bias"], ins["k_bias"], None, False, case["scale"], ins["do"],
        dtype=torch.float64)
    assert max_abs(o64, ref["o"]) < 1e-5
    assert max_abs(g64[0], ref["dq"]) < 5e-5


def test_oracle_row_blocking_is_exact():
    case, ins, _ = load_golden("causal_r2")
    a = orc.attention_forward_backward(ins["q"], ins["k"], ins["v"], ins["q_bias"], ins["k_bias"], None,
                                       True, case["scale"], ins["do"], block_rows=4096)
    b = orc.attention_forward_backward(ins["q"], ins["k"], ins["v"], ins["q_bias"], ins["k_bias"], None,
                                       True, case["scale"], ins["do"], block_rows=17)
    assert max_abs(a[0], b[0]) < 1e-6
    for x, y in zip(a[2], b[2]):
        assert max_abs(x, y) < 2e-5


def test_oracle_fully_masked_rows_are_zero():
    q = torch.randn(1, 4, 1, 16)
    k = torch.randn(1, 6, 1, 16)
    v = torch.randn(1, 6, 1, 16)
    mask = torch.zeros(1, 1, 4, 6)
    mask[0, 0, 2, :] = float("-inf")
    o, lse = orc.attention_forward(q, k, v, None, None, mask, False, None)
    assert torch.all(o[0, 2] == 0) and lse[0, 0, 2] == float("-inf")
    assert torch.isfinite(o).all()
