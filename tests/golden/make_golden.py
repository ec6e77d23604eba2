"""Generate golden vectors from the reference's own naive attention.

Run once in a container that has the reference checked out:

    python tests/golden/make_golden.py /path/to/reference

It imports ``attention_torch`` from the reference's ``flash_bias/attention_func.py``
(with stand-in modules for its GPU-only imports, which this path never calls),
evaluates it in fp32 on the CPU with the dense bias materialised from the factors
exactly as the reference's correctness script does, back-propagates a seeded dO with
autograd, and writes one ``.npz`` per case next to this file.  The test-suite only
reads the ``.npz`` files; the reference itself is not needed to run the tests.
"""
import math
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# name, B, Sq, Sk, H, D, R, causal, scale, bias-broadcast (batch, head), mask kind, input dtype
CASES = [
    ("c1_small",      2, 64, 64, 2, 32, 8, False, None, (False, False), None, torch.float16),
    ("causal_r2",     1, 96, 96, 3, 32, 2, True, None, (True, False), None, torch.bfloat16),
    ("ragged_cross",  2, 50, 77, 2, 16, 5, False, 0.5, (False, True), None, torch.bfloat16),
    ("causal_cross",  1, 70, 45, 2, 64, 3, True, None, (False, False), None, torch.float16),
    ("mask_vector",   2, 40, 56, 2, 32, 4, False, 1.0, (True, True), "vector", torch.float16),
    ("mask_matrix",   2, 33, 48, 3, 24, 16, False, None, (True, False), "matrix", torch.bfloat16),
    ("no_bias",       1, 48, 48, 2, 128, 0, True, None, (False, False), None, torch.bfloat16),
    ("benchmark_1k",  1, 256, 256, 2, 32, 8, False, None, (False, False), None, torch.float16),
]


def load_reference(ref_root):
    for name in ("xformers", "xformers.ops"):
        sys.modules.setdefault(name, types.ModuleType(name))
    sys.modules["xformers"].ops = sys.modules["xformers.ops"]
    sys.path.insert(0, os.path.join(ref_root, "flash_bias"))
    import attention_func  # noqa: E402
    return attention_func.attention_torch


def make_inputs(case):
    name, B, Sq, Sk, H, D, R, causal, scale, (bb, hb), mask_kind, dtype = case
    g = torch.Generator().manual_seed(sum(map(ord, name)))
    rn = lambda *s: torch.randn(*s, generator=g, dtype=torch.float32).to(dtype).float()
    t = dict(q=rn(B, Sq, H, D), k=rn(B, Sk, H, D), v=rn(B, Sk, H, D), do=rn(B, Sq, H, D))
    if R:
        t["q_bias"] = rn(1 if bb else B, Sq, 1 if hb else H, R)
        t["k_bias"] = rn(1 if bb else B, Sk, 1 if hb else H, R)
    if mask_kind == "vector":
        t["mask"] = rn(B, 1, 1, Sk)
    elif mask_kind == "matrix":
        t["mask"] = rn(1, H, Sq, Sk)
    return t


def main():
    attention_torch = load_reference(sys.argv[1])
    for case in CASES:
        name, B, Sq, Sk, H, D, R, causal, scale, _, mask_kind, dtype = case
        t = make_inputs(case)
        leaves = {n: t[n].clone().requires_grad_(True) for n in ("q", "k", "v", "q_bias", "k_bias") if n in t}
        sc = scale or 1.0 / math.sqrt(D)
        bias = None
        if R:
            # (B,H,Sq,Sk) dense bias, as flash_bias/benchmark.py:42-43
            bias = leaves["q_bias"].permute(0, 2, 1, 3) @ leaves["k_bias"].permute(0, 2, 1, 3).transpose(-2, -1)
            bias = bias.expand(B, H, Sq, Sk)
        if "mask" in t:
            m = t["mask"].expand(B, H, Sq, Sk)
            bias = m if bias is None else bias + m
        o = attention_torch(leaves["q"], leaves["k"], leaves["v"], sc, bias, causal)
        o.backward(t["do"])
        out = {"in_" + n: v.numpy() for n, v in t.items()}
        out["o"] = o.detach().numpy()
        for n, leaf in leaves.items():
            out["d" + n] = leaf.grad.numpy()
        out["meta"] = np.array([B, Sq, Sk, H, D, R, int(causal)], dtype=np.int64)
        out["scale"] = np.array([sc], dtype=np.float64)
        out["dtype"] = np.array([str(dtype)])
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
        print(name, "ok", {k: v.shape for k, v in out.items() if k.startswith("d") or k == "o"})


if __name__ == "__main__":
    main()
