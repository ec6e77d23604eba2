"""fb_fwd_noalloc: the forward entry point for hosts that may not allocate device memory inside the
call (plugin / custom-op hooks that receive only input and output buffers).  Its scratch is a fixed
array inside the library, so the test drives it through the C ABI without handing it any workspace
and compares with the regular entry point, twice in a row: the second call runs on top of whatever the
first left in the shared array.  Collected last on purpose."""
import ctypes as C

import pytest
import torch

from flashbias_b200 import _lib
from flashbias_b200.flash_bias import _fill_common, _strides_bhs, flash_bias_forward
from flashbias_b200.workloads import make_workload


def _params(w, o, lse):
    p = _lib.FbParams()
    _fill_common(p, w.q, w.k, w.v, w.q_bias, w.k_bias, None, w.causal, float(w.softmax_scale), 0)
    p.o, p.o_stride = o.data_ptr(), _strides_bhs(o)
    p.lse, p.lse_stride_bh = lse.data_ptr(), lse.shape[-1]
    return p


@pytest.mark.gpu
def test_noalloc_forward_matches_regular_forward_twice():
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    # two different problems back to back: different rank, head_dim and causal flag, so the second
    # call packs different factor widths over the first call's leftovers
    cases = [make_workload("alibi", B=1, H=4, S=640, D=32), make_workload("pde", B=2, H=2, S=1000, D=64)]
    for w in cases:
        w = w.to("cuda")
        o_ref, lse_ref, _ = flash_bias_forward(w.q, w.k, w.v, w.q_bias, w.k_bias, None, w.causal, w.softmax_scale)
        o = torch.full_like(w.q, float("nan"))
        lse = torch.full_like(lse_ref, float("nan"))
        p = _params(w, o, lse)
        assert lib.fb_fwd_workspace_bytes(C.byref(p)) > 0, "the case must actually need scratch"
        assert p.workspace is None and p.workspace_bytes == 0
        rc = lib.fb_fwd_noalloc(C.byref(p), stream)
        assert rc == 0, _lib.strerror(rc)
        torch.cuda.synchronize()
        # a second call of the same problem (the kernel variant and the scratch address are set up by now)
        # must leave the amount of free device memory untouched: nothing is allocated inside the call
        free0, _ = torch.cuda.mem_get_info()
        rc = lib.fb_fwd_noalloc(C.byref(p), stream)
        assert rc == 0, _lib.strerror(rc)
        torch.cuda.synchronize()
        free1, _ = torch.cuda.mem_get_info()
        assert free1 == free0, "fb_fwd_noalloc changed the free device memory"
        Sq = w.q.shape[1]
        assert (o.float() - o_ref.float()).abs().max().item() <= 2e-2
        assert (lse[..., :Sq] - lse_ref[..., :Sq]).abs().max().item() <= 2e-2
        assert torch.equal(o, o_ref), "same kernels, same inputs: the results should be identical"


def test_noalloc_rejects_problems_beyond_its_capacity():
    lib = _lib.load()
    cap = lib.fb_fwd_noalloc_capacity()
    assert cap == 32 << 20
    p = _lib.FbParams()
    p.B, p.H, p.Sq, p.Sk, p.D, p.R = 64, 64, 65536, 65536, 32, 8
    p.dtype = _lib.FB_DTYPE_BF16
    p.softmax_scale = 0.17
    for name in ("q", "k", "v", "o", "lse", "q_bias", "k_bias"):
        setattr(p, name, 0x1000)  # never dereferenced: the size check comes before any launch
    row, head = 64 * 32, 32
    for name in ("q_stride", "k_stride", "v_stride", "o_stride"):
        setattr(p, name, _lib.I64x3(65536 * row, head, row))
    for name in ("q_bias_stride", "k_bias_stride"):
        setattr(p, name, _lib.I64x3(65536 * 64 * 8, 8, 64 * 8))
    p.lse_stride_bh = 65536
    assert lib.fb_fwd_workspace_bytes(C.byref(p)) > cap
    assert lib.fb_fwd_noalloc(C.byref(p), None) == -11
    assert "scratch" in _lib.strerror(-11)
