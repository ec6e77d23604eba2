"""Tensor-core building blocks (TMA tiles, shared-memory descriptors, tcgen05 MMA, TMEM loads)
checked one operand-layout flavour at a time against a host matmul, through the C ABI."""
import ctypes as C

import pytest
import torch

from flashbias_b200 import _lib

pytestmark = pytest.mark.gpu


def _cases():
    try:
        return list(range(_lib.load().fb_selftest_count()))
    except Exception:
        return []


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case_id", _cases())
def test_umma_descriptor_flavour(case_id, dtype):
    lib = _lib.load()
    vals = [C.c_int32() for _ in range(7)]
    assert lib.fb_selftest_info(case_id, *[C.byref(v) for v in vals]) == 0
    a_rows, a_cols, b_rows, b_cols, n, a_t, b_t = (v.value for v in vals)
    g = torch.Generator().manual_seed(100 + case_id)
    a = torch.randn(a_rows, a_cols, generator=g).to(dtype).cuda()
    b = torch.randn(b_rows, b_cols, generator=g).to(dtype).cuda()
    d = torch.full((128, n), float("nan"), device="cuda", dtype=torch.float32)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    dt = _lib.FB_DTYPE_BF16 if dtype == torch.bfloat16 else _lib.FB_DTYPE_F16
    rc = lib.fb_selftest_run(case_id, dt, a.data_ptr(), b.data_ptr(), d.data_ptr(), status.data_ptr(),
                             torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _lib.strerror(rc)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    af, bf = a.float(), b.float()
    want = (af.t() if a_t else af) @ (bf.t() if b_t else bf)
    err = (d - want).abs().max().item()
    assert err < 1e-2 * max(1.0, want.abs().max().item() / 16), f"case {case_id}: max err {err}"
