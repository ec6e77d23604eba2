"""The host-buffer entry (chunked copies overlapped with the kernels) gives the results of one call on the whole
tensors: bit-identical where a single CTA produces the value (o, dk, dv), equal up to the order of the fp32
additions where several key tiles add into one accumulator (dq and the factor gradients)."""
import pytest
import torch

from flashbias_b200.flash_bias import flash_bias_backward, flash_bias_forward
from flashbias_b200.host_pipeline import HostPipeline
from flashbias_b200.workloads import make_workload

pytestmark = pytest.mark.gpu

CASES = {
    "alibi": (dict(B=1, H=24, S=2048, D=32), "head"),        # factors per head, shared over batch
    "pde": (dict(B=3, H=4, S=4096, D=64), "batch"),          # factors per batch entry, shared over heads
    "generic": (dict(B=2, H=24, S=2048, D=32, R=8), "head"),  # factors per (batch, head)
    "swin": (dict(B=32, H=24, window=16, D=32, R=16), "head"),
    "alibi_few_heads": (dict(B=1, H=6, S=4096, D=32), "none"),  # head chunks would be 128-byte rows: one chunk
    "pairformer": (dict(B=1, H=4, S=512, D=32, R=32), "none"),  # too small to be worth chunking
}


@pytest.mark.parametrize("name", list(CASES))
def test_pipeline_matches_single_call(name):
    sizes, dim = CASES[name]
    w = make_workload(name.split("_")[0], **sizes)
    names = ("q", "k", "v", "q_bias", "k_bias", "do")
    host_in = {n: t.pin_memory() for n, t in zip(names, (w.q, w.k, w.v, w.q_bias, w.k_bias, w.do))}
    like = {"o": w.q, "dq": w.q, "dk": w.k, "dv": w.v, "dq_bias": w.q_bias, "dk_bias": w.k_bias}
    host_out = {n: torch.full(t.shape, float("nan"), dtype=t.dtype).pin_memory() for n, t in like.items()}
    pipe = HostPipeline(host_in, "cuda", chunks=3)
    assert pipe.dim == dim and (len(pipe.ranges) > 1) == (dim != "none")
    for _ in range(2):  # buffers are reused from call to call
        pipe.run(host_in, host_out, w.causal, w.softmax_scale)

    d = w.to("cuda")
    o, lse, sc = flash_bias_forward(d.q, d.k, d.v, d.q_bias, d.k_bias, None, w.causal, w.softmax_scale)
    grads = flash_bias_backward(d.do, d.q, d.k, d.v, o, d.q_bias, d.k_bias, lse, None, w.causal, sc)
    torch.cuda.synchronize()
    want = dict(zip(("o", "dq", "dk", "dv", "dq_bias", "dk_bias"), (o,) + tuple(grads)))
    for key in ("o", "dk", "dv"):
        assert torch.equal(host_out[key], want[key].cpu()), key
    for key in ("dq", "dq_bias", "dk_bias"):
        got, ref = host_out[key].float(), want[key].cpu().float()
        assert not torch.isnan(got).any(), key
        # one unit in the last place of the 16-bit result, relative to the tensor's scale
        tol = 2.0 ** (-7 if got.dtype == torch.bfloat16 or w.dtype == torch.bfloat16 else -10) * ref.abs().max().clamp_min(1e-6)
        assert (got - ref).abs().max() <= tol, key
