#!/usr/bin/env python
"""Benchmark of the FlashBias hot path: forward + backward attention with a low-rank bias.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl flashbias|reference]
                    [--replicas] [--no-extras]

A step is one forward + backward pass of ``flash_bias_func`` over one synthetic batch of the named
workload (default ``alibi``: causal ALiBi attention, B1 H50 S8192 D32 R2, bf16).

With N > 1 the script is launched with one process per GPU (torchrun).  Default: ONE problem of the
workload is partitioned over the ranks by (batch, head) ranges (``flashbias_b200.sharding``), each rank
runs the operator on its slab, there is no collective in the timed region, and ``scaling`` is "strong"
(total work fixed).  Factor gradients of factors that ranks share need one sum across ranks afterwards;
it is timed separately.  ``--replicas`` gives every rank an independent whole problem instead ("weak").

Printed: ONE JSON line with the metric (algorithmic TFLOP/s, T*(14D+8R) flop per step with T the
number of attended (query, key) pairs), the device-timed ms/step, the same metric end to end from
pinned host buffers (``e2e``), the roofline of the dominant kernel (backward main kernel, timed with
CUDA events around each of its launches inside the library), the CPU baseline, and -- at N = 1 --
sub-records for the fused ALiBi producer, for the other four benchmark workloads and for the reference's
Triton kernel on the same GPU.

``--impl reference`` times the CPU restatement of the reference's naive attention on the host cores
on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from flashbias_b200.workloads import (alibi_slopes, flops_bwd, flops_fwd, make_device_workload,  # noqa: E402
                                      make_workload, swin_shift_mask)

FULL_SIZES = {
    "generic": dict(B=2, H=4, S=1024, D=32, R=8),
    "alibi": dict(B=1, H=50, S=8192, D=32),
    "swin": dict(B=4096, H=24, window=16, D=32, R=16),
    "pde": dict(B=2, H=8, S=32768, D=64),
    "pairformer": dict(B=1, H=16, S=1536, D=32, R=32),
}
# reduced cases for profiler captures (--profile-case): same kernels, inputs larger than L2, a few hundred MB at most
PROFILE_SIZES = {
    "generic": dict(B=2, H=4, S=1024, D=32, R=8),
    "alibi": dict(B=1, H=16, S=4096, D=32),
    "swin": dict(B=256, H=24, window=16, D=32, R=16),
    "pde": dict(B=1, H=4, S=8192, D=64),
    "pairformer": dict(B=1, H=16, S=1536, D=32, R=32),
}
# bounded CPU sample of each workload: (sizes of the sample, how it scales to the full workload)
CPU_SAMPLE = {
    "generic": (dict(B=2, H=4, S=1024, D=32, R=8), "whole workload"),
    "alibi": (dict(B=1, H=2, S=8192, D=32), "2 of 50 heads"),
    "swin": (dict(B=32, H=24, window=16, D=32, R=16), "32 of 4096 windows"),
    "pde": (dict(B=1, H=1, S=8192, D=64), "1 head of 8192 points (1/16 of the rows and keys)"),
    "pairformer": (dict(B=1, H=4, S=1536, D=32, R=32), "4 of 16 heads"),
}

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the backward main kernel, per workload: taken from
# the ncu captures of the reduced cases (PROFILE_SIZES, `--profile-case`) and scaled to the full workload by the
# number of (batch, head, row) units - the tiles a CTA re-streams (Q, dO per key tile) are served by L2 at both
# sizes, so DRAM traffic grows with the rows, not with the tile pairs
NCU_BWD_TRAFFIC_BYTES = {
    "alibi": (47.8e6 + 0.121e6) * (50 * 8192) / (16 * 4096),
    "swin": (839.7e6 + 381.7e6) * 4096 / 256,
    "pde": 27.64e6 * (2 * 8 * 32768) / (4 * 8192),
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(bf16_tflops=float(d["bf16_tflops"]), hbm_gbs=float(d["hbm_gbs"]), source="measured")
    return dict(bf16_tflops=1590.0, hbm_gbs=6650.0, source="fallback")


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU with NVML while the timed region runs."""

    def __init__(self, index: int, period: float = 0.02):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._halt = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._halt.wait(self.period)

    def stop(self):
        self._halt.set()
        self.join(timeout=2)
        s = sorted(self.samples)
        med = s[len(s) // 2] if s else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(s)}


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


def workload_config(name, causal, rank_dim):
    """The `config` keys both arms share."""
    return {"workload": name, **FULL_SIZES[name], "causal": causal, "rank": rank_dim}


def flops_of(sh, causal):
    return (flops_fwd(sh["B"], sh["H"], sh["Sq"], sh["Sk"], sh["D"], sh["R"], causal),
            flops_bwd(sh["B"], sh["H"], sh["Sq"], sh["Sk"], sh["D"], sh["R"], causal))


def bwd_bytes(sh, nfac):
    """Algorithmic bytes of one backward call: reads q,k,v,o,dO,factors,lse,delta; writes dq,dk,dv,dq_bias,dk_bias."""
    return 2 * (sh["B"] * sh["H"] * (4 * sh["Sq"] * sh["D"] + 4 * sh["Sk"] * sh["D"]) + 2 * nfac) + \
        8 * sh["B"] * sh["H"] * sh["Sq"]


def cpu_baseline(workload, max_seconds=10.0, max_passes=5):
    """The CPU restatement of the reference's naive attention on a bounded sample, all host threads."""
    from oracle import flashbias_oracle as orc
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cs, what = CPU_SAMPLE[workload]
    cw = make_workload(workload, **cs)
    cf, cb = flops_of(cw.shape, cw.causal)
    f32 = [t.float() for t in (cw.q, cw.k, cw.v, cw.q_bias, cw.k_bias)]
    t0 = time.perf_counter()
    n = 0
    while n < 1 or (time.perf_counter() - t0 < max_seconds and n < max_passes):
        orc.attention_forward_backward(*f32, None, cw.causal, cw.softmax_scale, cw.do.float())
        n += 1
    cdt = (time.perf_counter() - t0) / n
    return {"value": (cf + cb) / cdt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"{what}, {n} pass(es) of {cdt:.2f} s; fp32 naive attention with the bias materialised, "
                      "torch CPU ops"}, cdt


def run_reference(args, rank):
    """CPU arm: the restated naive attention on the host cores, bounded sample per step."""
    if rank != 0:
        return
    from oracle import flashbias_oracle as orc
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    sizes, what = CPU_SAMPLE[args.workload]
    w = make_workload(args.workload, **sizes)
    ff, fb = flops_of(w.shape, w.causal)
    f32 = [t.float() for t in (w.q, w.k, w.v, w.q_bias, w.k_bias)]

    def step():
        orc.attention_forward_backward(*f32, None, w.causal, w.softmax_scale, w.do.float())

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    val = (ff + fb) / dt / 1e12
    line = {
        "impl": "reference", "metric": "fwd+bwd attention TFLOP/s", "value": val, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak" if args.replicas else "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.workload, w.causal, w.shape["R"]),
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": f"{what}; fp32 naive attention with the bias materialised, torch CPU ops"},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


class Timer:
    """Device timing of a callable: CUDA events per call, L2 flushed (256 MiB write) between calls; the main
    kernels are also timed inside the library (events around each launch of one kernel class)."""

    def __init__(self, lib, dev):
        self.lib = lib
        self.flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)  # > 126 MB L2

    def run(self, fn, n, kernel_class=0):
        if kernel_class:
            self.lib.fb_prof_begin(kernel_class)
        evs = []
        for _ in range(n):
            self.flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            evs.append((a, b))
        torch.cuda.synchronize()
        ms = sum(a.elapsed_time(b) for a, b in evs) / n
        kms, kn = C.c_float(), C.c_int()
        if kernel_class:
            self.lib.fb_prof_end(C.byref(kms), C.byref(kn))
        return ms, (kms.value / kn.value if kn.value else None), kn.value


def rooflines(peaks, fl_b, bytes_b, bwd_kernel_ms):
    """Tensor and HBM fractions of the backward main kernel from its algorithmic flop / bytes; the binding one is
    the roofline with the larger lower bound on the kernel's time."""
    if not bwd_kernel_ms:
        return None, None, None
    t = bwd_kernel_ms * 1e-3
    ach = fl_b / t / 1e12
    gbs = bytes_b / t / 1e9
    tensor = {"achieved": ach, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": ach / peaks["bf16_tflops"]}
    hbm = {"achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"]}
    hbm_binds = bytes_b / (peaks["hbm_gbs"] * 1e9) > fl_b / (peaks["bf16_tflops"] * 1e12)
    return tensor, hbm, hbm_binds


def sub_record(timer, fn_fwd, fn_step, ff, fb, bytes_b, peaks, n):
    """ms / TFLOP/s / roofline fractions of one operator variant on one workload (device-timed)."""
    for _ in range(3):
        fn_step()
    torch.cuda.synchronize()
    ms_step, bwd_k, _ = timer.run(fn_step, n, 2)
    with torch.no_grad():
        fwd_ms, fwd_k, _ = timer.run(fn_fwd, max(3, n // 2), 1)
    tensor, hbm, hbm_binds = rooflines(peaks, fb, bytes_b, bwd_k)
    rec = {"ms_per_step": ms_step, "tflops": (ff + fb) / (ms_step * 1e-3) / 1e12, "fwd_ms": fwd_ms,
           "fwd_kernel_ms": fwd_k, "fwd_kernel_tflops": ff / (fwd_k * 1e-3) / 1e12 if fwd_k else None,
           "fwd_kernel_frac_of_bf16_peak": ff / (fwd_k * 1e-3) / 1e12 / peaks["bf16_tflops"] if fwd_k else None,
           "bwd_kernel_ms": bwd_k}
    if tensor:
        rec.update({"bwd_kernel_tflops": tensor["achieved"], "bwd_tensor_frac": tensor["frac"],
                    "bwd_hbm_gbs": hbm["achieved"], "bwd_hbm_frac": hbm["frac"],
                    "binding": "hbm" if hbm_binds else "tensor",
                    "step_frac_of_bf16_peak": rec["tflops"] / peaks["bf16_tflops"]})
    return rec


def triton_baseline(w, d, timer, o_ours, n):
    """The reference's Triton kernel (unmodified file under baseline/_ref) on the same GPU and inputs: parity of
    its forward against this library's, then forward and forward+backward times.  Returns the failure text
    instead if the file is absent or Triton cannot build or run it here."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.exists(os.path.join(ref_dir, "flash_bias_triton.py")):
        return {"unavailable": "baseline/_ref/flash_bias_triton.py is not present on this machine"}
    try:
        sys.path.insert(0, ref_dir)
        import flash_bias_triton
        fn = flash_bias_triton.flash_bias_func
        sh = w.shape
        q, k, v = (t.clone().requires_grad_(True) for t in (d.q, d.k, d.v))
        # the reference's backward indexes factors with un-expanded strides: give it expanded, contiguous factors
        qb = d.q_bias.expand(sh["B"], -1, sh["H"], -1).contiguous().requires_grad_(True)
        kb = d.k_bias.expand(sh["B"], -1, sh["H"], -1).contiguous().requires_grad_(True)

        def fwd():
            return fn(q, k, v, qb, kb, None, w.causal, w.softmax_scale)

        def step():
            fwd().backward(d.do)

        with torch.no_grad():
            o_t = fwd()
        torch.cuda.synchronize()
        dev_o = float((o_t.float() - o_ours.float()).abs().max())
        for _ in range(2):
            step()
        torch.cuda.synchronize()
        ms_step, _, _ = timer.run(step, n)
        with torch.no_grad():
            fwd_ms, _, _ = timer.run(fwd, n)
        ff, fb = flops_of(sh, w.causal)
        return {"kernel": "flash_bias/flash_bias_triton.py (reference, unmodified)", "triton": __import__("triton").__version__,
                "fwd_ms": fwd_ms, "fwd_tflops": ff / (fwd_ms * 1e-3) / 1e12, "ms_per_step": ms_step,
                "tflops": (ff + fb) / (ms_step * 1e-3) / 1e12, "fwd_max_abs_vs_this_library": dev_o,
                "note": "its bias dot runs in TF32: on ALiBi-sized factors its forward is off by whole units"}
    except Exception as e:  # recorded, not raised: the baseline is context, not the product
        return {"failed": f"{type(e).__name__}: {str(e)[:300]}"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="alibi", choices=sorted(FULL_SIZES))
    ap.add_argument("--impl", default="flashbias", choices=["flashbias", "reference"])
    ap.add_argument("--replicas", action="store_true",
                    help="N > 1: every rank runs an independent whole problem (weak scaling) instead of a slab of one")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the sub-records (producer path, other workloads, Triton and CPU baselines)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile-case", action="store_true",
                    help="run only --steps forward+backward calls of a reduced case (for a profiler capture); "
                         "prints no bench line")
    ap.add_argument("--producer", action="store_true", help="with --profile-case: use the fused ALiBi producer")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "flashbias" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch.distributed as dist
    from flashbias_b200 import _lib, flash_bias_alibi_func, flash_bias_func
    from flashbias_b200.sharding import allreduce_shared_factor_grads, bh_slabs, shared_factor_flags

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # NCCL's own messages (its version line among them) go to stderr: stdout carries the one JSON line
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()

    if args.profile_case:
        w = make_workload(args.workload, **PROFILE_SIZES[args.workload]).to(dev)
        q, k, v, qb, kb = (t.requires_grad_(True) for t in (w.q, w.k, w.v, w.q_bias, w.k_bias))
        sl = alibi_slopes(w.shape["H"]).to(dev)
        for _ in range(args.warmup + args.steps):
            if args.producer:
                flash_bias_alibi_func(q, k, v, sl, w.causal, w.softmax_scale).backward(w.do)
            else:
                flash_bias_func(q, k, v, qb, kb, None, w.causal, w.softmax_scale).backward(w.do)
        torch.cuda.synchronize()
        print(json.dumps({"profile_case": args.workload, **PROFILE_SIZES[args.workload]}), flush=True)
        return

    sizes = FULL_SIZES[args.workload]
    w = make_workload(args.workload, **sizes)  # every rank draws the same seeded problem on its host
    sh = w.shape
    B, H = sh["B"], sh["H"]
    fl_f, fl_b = flops_of(sh, w.causal)
    sharded = world > 1 and not args.replicas
    slabs = bh_slabs(B, H, rank, world) if sharded else [(0, B, 0, H)]

    def cut(t, slab, pin=False):
        """This rank's part of a (B|1, S, H|1, C) host tensor for one slab, contiguous."""
        b0, b1, h0, h1 = slab
        bs = slice(0, 1) if t.shape[0] == 1 else slice(b0, b1)
        hs = slice(0, 1) if t.shape[2] == 1 else slice(h0, h1)
        out = t[bs, :, hs].contiguous()
        return out.pin_memory() if pin else out

    names = ("q", "k", "v", "q_bias", "k_bias", "do")
    host_slabs = [{n: cut(getattr(w, n), s, pin=True) for n in names} for s in slabs]
    dev_slabs = []
    for hs in host_slabs:
        d = {n: t.to(dev) for n, t in hs.items()}
        for n in ("q", "k", "v", "q_bias", "k_bias"):
            d[n].requires_grad_(True)
        dev_slabs.append(d)
    timer = Timer(lib, dev)

    def step():
        outs = []
        for d in dev_slabs:
            for n in ("q", "k", "v", "q_bias", "k_bias"):
                d[n].grad = None
            o = flash_bias_func(d["q"], d["k"], d["v"], d["q_bias"], d["k_bias"], None, w.causal, w.softmax_scale)
            o.backward(d["do"])
            outs.append(o)
        return outs

    def fwd_only():
        for d in dev_slabs:
            flash_bias_func(d["q"], d["k"], d["v"], d["q_bias"], d["k_bias"], None, w.causal, w.softmax_scale)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()

    # ---- timed region: K steps, device-timed per step, L2 flushed between steps
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    launches0 = lib.fb_launch_count()
    barrier()
    ms_step, bwd_kernel_ms, kn = timer.run(step, args.steps, 2)
    barrier()
    launches = lib.fb_launch_count() - launches0
    clocks = sampler.stop()
    if bwd_kernel_ms is not None:
        bwd_kernel_ms *= len(dev_slabs)  # per step of this rank (one launch per slab)

    with torch.no_grad():
        fwd_ms, fwd_kernel_ms, _ = timer.run(fwd_only, max(3, args.steps // 2), 1)
    if fwd_kernel_ms is not None:
        fwd_kernel_ms *= len(dev_slabs)

    # ---- the one exchange step of the partition: sum of the gradients of factors that ranks share
    allreduce_ms = None
    if sharded:
        q_shared, k_shared = shared_factor_flags(B, H, tuple(w.q_bias.shape), tuple(w.k_bias.shape), world)
        if q_shared or k_shared:
            dqb = torch.zeros(w.q_bias.shape, dtype=torch.float32, device=dev)
            dkb = torch.zeros(w.k_bias.shape, dtype=torch.float32, device=dev)
            for _ in range(3):
                allreduce_shared_factor_grads(dqb, dkb, q_shared, k_shared)
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(10):
                allreduce_shared_factor_grads(dqb, dkb, q_shared, k_shared)
            b.record()
            torch.cuda.synchronize()
            allreduce_ms = a.elapsed_time(b) / 10

    # ---- end to end: pinned host inputs -> device, fwd+bwd, results -> host, every step
    from flashbias_b200.host_pipeline import HostPipeline
    h2d = d2h = 0
    pipes = []
    for hs in host_slabs:
        out_like = {"o": hs["q"], "dq": hs["q"], "dk": hs["k"], "dv": hs["v"], "dq_bias": hs["q_bias"],
                    "dk_bias": hs["k_bias"]}
        out_host = {n: torch.empty(t.shape, dtype=t.dtype).pin_memory() for n, t in out_like.items()}
        pipes.append((HostPipeline(hs, dev), hs, out_host))
        h2d += sum(t.numel() * t.element_size() for t in hs.values())
        d2h += sum(t.numel() * t.element_size() for t in out_host.values())
    e2e_steps = max(3, min(args.steps, 20))

    def e2e_step():
        for pipe, hs, out_host in pipes:
            pipe.run(hs, out_host, w.causal, w.softmax_scale)

    e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps

    # ---- shard check (outside the timed region): this rank's slab of a whole-problem run on this GPU
    shard_check = None
    if sharded:
        full = w.to(dev)
        fq, fk, fv, fqb, fkb = (t.requires_grad_(True) for t in (full.q, full.k, full.v, full.q_bias, full.k_bias))
        fo = flash_bias_func(fq, fk, fv, fqb, fkb, None, w.causal, w.softmax_scale)
        fo.backward(full.do)
        outs = step()
        torch.cuda.synchronize()
        same, dq_err = True, 0.0
        for (b0, b1, h0, h1), d, o in zip(slabs, dev_slabs, outs):
            same &= torch.equal(o, fo[b0:b1, :, h0:h1])
            same &= torch.equal(d["k"].grad, fk.grad[b0:b1, :, h0:h1])
            same &= torch.equal(d["v"].grad, fv.grad[b0:b1, :, h0:h1])
            dq_err = max(dq_err, float((d["q"].grad.float() - fq.grad[b0:b1, :, h0:h1].float()).abs().max()))
        flag = torch.tensor([1.0 if same else 0.0, -dq_err], device=dev, dtype=torch.float64)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        shard_check = {"o_dk_dv_bit_identical_to_one_gpu_run": bool(flag[0].item() == 1.0),
                       "dq_max_abs_vs_one_gpu_run": float(-flag[1].item()),
                       "note": "dq is an fp32 sum over key tiles whose order of addition is not fixed"}
        del full, fq, fk, fv, fqb, fkb, fo

    stats = torch.tensor([ms_step, e2e_ms, fwd_ms, bwd_kernel_ms or 0.0, fwd_kernel_ms or 0.0], device=dev,
                         dtype=torch.float64)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    ms_step, e2e_ms, fwd_ms, bwd_kernel_ms, fwd_kernel_ms = (float(x) for x in stats.cpu())
    totals = torch.tensor([float(launches), float(h2d), float(d2h)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(totals, op=dist.ReduceOp.SUM)
    launches, h2d, d2h = (int(x) for x in totals.cpu())

    if rank == 0:
        peaks = load_peaks()
        fl = fl_f + fl_b
        problems = world if (world > 1 and not sharded) else 1  # whole problems in the job
        value = problems * fl / (ms_step * 1e-3) / 1e12
        # roofline of the dominant kernel: rank 0's slab (the largest one) of the backward main kernel
        b0, b1, h0, h1 = slabs[0]
        frac_r0 = sum((s[1] - s[0]) * (s[3] - s[2]) for s in slabs) / (B * H)
        nfac = (w.q_bias.numel() + w.k_bias.numel()) if w.q_bias is not None else 0
        tensor, hbm, hbm_binds = rooflines(peaks, fl_b * frac_r0, bwd_bytes(sh, nfac) * frac_r0, bwd_kernel_ms)
        # (bwd_sm100_kernel; its persistent form bwd_p_sm100_kernel where a work item has few query tiles)
        roof = {"bound": "hbm" if hbm_binds else "tensor", "kernel": "bwd_sm100_kernel",
                **((hbm if hbm_binds else tensor) or {}), "peak_source": peaks["source"],
                "ms_per_step_in_kernel": bwd_kernel_ms, "launches_timed": kn, "flop_per_step": fl_b * frac_r0,
                "bytes_per_step": bwd_bytes(sh, nfac) * frac_r0, "other_roofline": tensor if hbm_binds else hbm,
                "traffic": NCU_BWD_TRAFFIC_BYTES.get(args.workload) if world == 1 else None}
        # the reference's own flop convention (benchmark.py: (4D+1) B H S^2 forward, x3 forward+backward, no
        # causal discount), so that numbers can be laid beside its tables
        ref_fl = 3.0 * (4 * sh["D"] + 1) * sh["B"] * sh["H"] * sh["Sq"] * sh["Sk"]
        line = {
            "metric": "fwd+bwd attention TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong" if sharded or world == 1 else "weak", "vs_baseline": None,
            "dtype": "bf16" if w.dtype == torch.bfloat16 else "f16", "data": "synthetic",
            "config": workload_config(args.workload, w.causal, sh["R"]),
            "detail": {"partition": ("one problem, (batch, head) slabs per rank: " + str(slabs) + " on rank 0"
                                     if sharded else ("independent replicas" if world > 1 else "one GPU")),
                       "l2": "flushed between steps (256 MiB write)",
                       "fwd_ms": fwd_ms, "fwd_tflops": problems * fl_f / (fwd_ms * 1e-3) / 1e12,
                       "fwd_kernel_ms": fwd_kernel_ms,
                       "fwd_kernel_tflops": fl_f * frac_r0 / (fwd_kernel_ms * 1e-3) / 1e12 if fwd_kernel_ms else None,
                       "fwd_kernel_frac_of_bf16_peak": (fl_f * frac_r0 / (fwd_kernel_ms * 1e-3) / 1e12 /
                                                        peaks["bf16_tflops"]) if fwd_kernel_ms else None,
                       "step_frac_of_bf16_peak": value / (world * peaks["bf16_tflops"]),
                       "flop_convention": "T*(14D+8R), T = attended (query,key) pairs",
                       "reference_convention_tflops": problems * ref_fl / (ms_step * 1e-3) / 1e12,
                       "factor_grad_allreduce_ms": allreduce_ms},
            "clocks": clocks,
            "e2e": {"value": problems * fl / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": int(launches),
            "roofline": roof,
        }
        if shard_check is not None:
            line["shard_check"] = shard_check
        if world == 1 and not args.no_extras:
            n_sub = max(5, min(args.steps, 20))
            d0 = dev_slabs[0]
            if args.workload == "alibi":
                # the same attention through the fused producer: slopes in, no factor tensors, dq/dk/dv out
                sl = alibi_slopes(H).to(dev)
                pq, pk, pv = (d0[n].detach().clone().requires_grad_(True) for n in ("q", "k", "v"))

                def p_fwd():
                    flash_bias_alibi_func(pq, pk, pv, sl, True, w.softmax_scale)

                def p_step():
                    for t in (pq, pk, pv):
                        t.grad = None
                    flash_bias_alibi_func(pq, pk, pv, sl, True, w.softmax_scale).backward(d0["do"])

                line["detail"]["alibi_producer"] = sub_record(timer, p_fwd, p_step, fl_f, fl_b,
                                                              bwd_bytes(sh, 0), peaks, n_sub)
            with torch.no_grad():
                o_ours = flash_bias_func(d0["q"], d0["k"], d0["v"], d0["q_bias"], d0["k_bias"], None, w.causal,
                                         w.softmax_scale)
            wd = type("W", (), {})()
            wd.q, wd.k, wd.v, wd.q_bias, wd.k_bias, wd.do = (d0[n].detach() for n in names)
            line["triton_baseline"] = triton_baseline(w, wd, timer, o_ours, max(3, min(args.steps, 10)))
            del o_ours
            others = {}
            for name in FULL_SIZES:
                if name == args.workload:
                    continue
                ow = make_device_workload(name, dev, **FULL_SIZES[name])
                osh = ow.shape
                off, ofb = flops_of(osh, ow.causal)
                oq, ok_, ov, oqb, okb = (t.requires_grad_(True) for t in (ow.q, ow.k, ow.v, ow.q_bias, ow.k_bias))

                def o_fwd():
                    flash_bias_func(oq, ok_, ov, oqb, okb, None, ow.causal, ow.softmax_scale)

                def o_step():
                    for t in (oq, ok_, ov, oqb, okb):
                        t.grad = None
                    flash_bias_func(oq, ok_, ov, oqb, okb, None, ow.causal, ow.softmax_scale).backward(ow.do)

                rec = sub_record(timer, o_fwd, o_step, off, ofb, bwd_bytes(osh, oqb.numel() + okb.numel()), peaks,
                                 max(3, n_sub // (4 if name in ("swin", "pde") else 1)))
                others[name] = {**FULL_SIZES[name], "causal": ow.causal, **rec}
                if name == "swin":
                    # the same workload as a shifted-window block: additive 0 / -100 mask of 64 entries, read as
                    # b % 64 by the kernels
                    smask = swin_shift_mask(FULL_SIZES[name]["window"], 8).to(dev)

                    def m_fwd():
                        flash_bias_func(oq, ok_, ov, oqb, okb, smask, ow.causal, ow.softmax_scale)

                    def m_step():
                        for t in (oq, ok_, ov, oqb, okb):
                            t.grad = None
                        flash_bias_func(oq, ok_, ov, oqb, okb, smask, ow.causal, ow.softmax_scale).backward(ow.do)

                    mbytes = bwd_bytes(osh, oqb.numel() + okb.numel()) + smask.numel() * 4
                    rec = sub_record(timer, m_fwd, m_step, off, ofb, mbytes, peaks, max(3, n_sub // 4))
                    others["swin_shifted"] = {**FULL_SIZES[name], "causal": ow.causal, "mask": "(64, 1, 256, 256) fp32",
                                              **rec}
                    del smask
                del ow, oq, ok_, ov, oqb, okb
                torch.cuda.empty_cache()
            line["detail"]["other_workloads"] = others
        if world == 1 and not args.no_cpu_baseline and not args.no_extras:
            line["cpu_baseline"], _ = cpu_baseline(args.workload)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
