"""What the reference's own contract costs in bf16, measured on the CPU in fp64.

The reference kernel rounds P to the 16-bit type before P.V and P^T.dO, and dS before its four products
(flash_bias/flash_bias_triton.py:317, :696, :714).  An implementation that does everything else exactly
(fp64 here) but keeps those roundings is already further from the fp32 checker (rounded to the output type)
than a relative L2 of 1e-3 when the type is bf16: the 1e-3 bound is attainable for fp16 only.  The GPU
parity tests therefore gate bf16 at 4e-3 (tests/helpers.py); this test pins the evidence for that number:
the floor is above 1e-3 and below 4e-3 on benchmark-like data."""
import pytest
import torch

from flashbias_b200.workloads import make_workload
from oracle import flashbias_oracle as orc
from tests.helpers import rel_l2


@pytest.mark.parametrize("name,sizes", [
    ("generic", dict(B=1, H=2, S=512, D=32, R=8, dtype=torch.bfloat16)),
    ("pde", dict(B=1, H=1, S=1024, D=64)),
    ("swin", dict(B=2, H=4, window=16, D=32, R=16)),
])
def test_bf16_rounding_of_p_and_ds_alone_exceeds_1e_3(name, sizes):
    w = make_workload(name, **sizes)
    assert w.dtype == torch.bfloat16
    f32 = [t.float() for t in (w.q, w.k, w.v, w.q_bias, w.k_bias)]
    do = w.do.float()
    # the fp32 checker, as the GPU tests use it
    o32, lse32 = orc.attention_forward(*f32, None, w.causal, w.softmax_scale)
    g32 = orc.attention_backward(do, *f32[:3], o32.to(w.dtype).float(), lse32, f32[3], f32[4], None, w.causal,
                                 w.softmax_scale)
    # exact arithmetic (fp64) with only the contract's roundings of P and dS, output rounded to bf16
    f64 = torch.float64
    o64, lse64 = orc.attention_forward(*f32, None, w.causal, w.softmax_scale, dtype=f64, round_p=w.dtype)
    g64 = orc.attention_backward(do, *f32[:3], o32.to(w.dtype).float(), lse64, f32[3], f32[4], None, w.causal,
                                 w.softmax_scale, dtype=f64, round_p=w.dtype)
    floors = {"o": rel_l2(o64.to(w.dtype).float(), o32.to(w.dtype).float())}
    for key, a, b in zip(("dq", "dk", "dv", "dq_bias", "dk_bias"), g64, g32):
        floors[key] = rel_l2(a.to(w.dtype).float(), b.to(w.dtype).float())
    print(name, {k: f"{v:.2e}" for k, v in floors.items()})
    # dq_bias = dS.k_bias cancels heavily against large, slowly varying factors: its floor is higher still (the
    # tensor-core backward evaluates it around a per-group centre for that reason and lands below this floor)
    for key, val in floors.items():
        assert val > 1e-3, f"{key}: bf16 floor {val:.2e}: the 1e-3 bound would be attainable after all"
        if key != "dq_bias":
            assert val < 4e-3, f"{key}: bf16 floor {val:.2e} is above the gate the GPU tests use"
