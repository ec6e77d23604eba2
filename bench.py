#!/usr/bin/env python
"""Benchmark of the FlashBias hot path: forward + backward attention with a low-rank bias.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl flashbias|reference]

A step is one forward + backward pass of ``flash_bias_func`` over one synthetic batch of the named
workload (default ``alibi``: causal ALiBi attention, B1 H50 S8192 D32 R2, bf16).  With N > 1 the
script is launched with one process per GPU (torchrun); every rank owns an independent batch of the
same shape (the path shards over batch x heads with no exchange step), so scaling is "weak" and the
reported value is the whole-job aggregate.

Printed: ONE JSON line with the metric (algorithmic TFLOP/s, T*(14D+8R) flop per step with T the
number of attended (query, key) pairs), the device-timed ms/step, the same metric end to end from
pinned host buffers (``e2e``), the roofline of the dominant kernel (backward main kernel, timed with
CUDA events around each of its launches inside the library), and the CPU baseline.

``--impl reference`` times the CPU restatement of the reference's naive attention on the host cores
on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from flashbias_b200.workloads import flops_bwd, flops_fwd, make_workload  # noqa: E402

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


# DRAM bytes (read + write) per launch of the backward main kernel, measured with ncu on this workload
NCU_BWD_TRAFFIC_BYTES = {"alibi": 1085593088 + 432811776}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(bf16_tflops=float(d["bf16_tflops"]), hbm_gbs=float(d["hbm_gbs"]), source="measured")
    return dict(bf16_tflops=1590.0, hbm_gbs=6650.0, source="fallback")


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU with NVML while the timed region runs."""

    def __init__(self, index: int, period: float = 0.1):
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
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


def run_reference(args, rank):
    """CPU arm: the restated naive attention on the host cores, bounded sample per step."""
    if rank != 0:
        return
    from oracle import flashbias_oracle as orc
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    sizes, what = CPU_SAMPLE[args.workload]
    w = make_workload(args.workload, **sizes)
    sh = w.shape
    fl = flops_fwd(sh["B"], sh["H"], sh["Sq"], sh["Sk"], sh["D"], sh["R"], w.causal) + \
        flops_bwd(sh["B"], sh["H"], sh["Sq"], sh["Sk"], sh["D"], sh["R"], w.causal)
    f32 = [t.float() for t in (w.q, w.k, w.v, w.q_bias, w.k_bias)]

    def step():
        orc.attention_forward_backward(*f32, None, w.causal, w.softmax_scale, w.do.float())

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    val = fl / dt / 1e12
    full = FULL_SIZES[args.workload]
    line = {
        "impl": "reference", "metric": "fwd+bwd attention TFLOP/s", "value": val, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, **full, "sample": what},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": f"{what}; fp32 naive attention with the bias materialised, torch CPU ops"},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="alibi", choices=sorted(FULL_SIZES))
    ap.add_argument("--impl", default="flashbias", choices=["flashbias", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile-case", action="store_true",
                    help="run only --steps forward+backward calls of a reduced case (for a profiler capture); "
                         "prints no bench line")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "flashbias" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch.distributed as dist
    from flashbias_b200 import _lib, flash_bias_func

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()

    if args.profile_case:
        w = make_workload(args.workload, **PROFILE_SIZES[args.workload]).to(dev)
        q, k, v, qb, kb = (t.requires_grad_(True) for t in (w.q, w.k, w.v, w.q_bias, w.k_bias))
        for _ in range(args.warmup + args.steps):
            flash_bias_func(q, k, v, qb, kb, None, w.causal, w.softmax_scale).backward(w.do)
        torch.cuda.synchronize()
        print(json.dumps({"profile_case": args.workload, **PROFILE_SIZES[args.workload]}), flush=True)
        return
    sizes = FULL_SIZES[args.workload]
    w = make_workload(args.workload, **sizes)
    sh = w.shape
    fl_f = flops_fwd(sh["B"], sh["H"], sh["Sq"], sh["Sk"], sh["D"], sh["R"], w.causal)
    fl_b = flops_bwd(sh["B"], sh["H"], sh["Sq"], sh["Sk"], sh["D"], sh["R"], w.causal)
    host = [t.pin_memory() for t in (w.q, w.k, w.v, w.q_bias, w.k_bias, w.do)]
    d = w.to(dev)
    q, k, v, qb, kb = (t.requires_grad_(True) for t in (d.q, d.k, d.v, d.q_bias, d.k_bias))
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)  # > 126 MB L2

    def step():
        for t in (q, k, v, qb, kb):
            t.grad = None
        o = flash_bias_func(q, k, v, qb, kb, None, w.causal, w.softmax_scale)
        o.backward(d.do)
        return o

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
    lib.fb_prof_begin(2)
    evs = []
    barrier()
    for _ in range(args.steps):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        step()
        b.record()
        evs.append((a, b))
    barrier()
    ms_total = sum(a.elapsed_time(b) for a, b in evs)
    import ctypes as C
    kms, kn = C.c_float(), C.c_int()
    lib.fb_prof_end(C.byref(kms), C.byref(kn))
    launches = lib.fb_launch_count() - launches0
    clocks = sampler.stop()

    # forward-only timing (reported in config for context)
    lib.fb_prof_begin(1)
    fe = []
    with torch.no_grad():
        for _ in range(max(3, args.steps // 2)):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            flash_bias_func(q, k, v, qb, kb, None, w.causal, w.softmax_scale)
            b.record()
            fe.append((a, b))
    torch.cuda.synchronize()
    fwd_ms = sum(a.elapsed_time(b) for a, b in fe) / len(fe)
    fkms, fkn = C.c_float(), C.c_int()
    lib.fb_prof_end(C.byref(fkms), C.byref(fkn))

    # ---- end to end: pinned host inputs -> device, fwd+bwd, results -> host, every step
    h2d = sum(t.numel() * t.element_size() for t in host)
    e2e_steps = max(3, min(args.steps, 10))

    # host tensors in, host tensors out, through the package's host entry: heads (or batch entries) are cut into
    # chunks whose copies overlap the kernels of the neighbouring chunks; every copy is inside the timed region
    from flashbias_b200.host_pipeline import HostPipeline
    names = ("q", "k", "v", "q_bias", "k_bias", "do")
    host_in = dict(zip(names, host))
    out_like = {"o": w.q, "dq": w.q, "dk": w.k, "dv": w.v, "dq_bias": w.q_bias, "dk_bias": w.k_bias}
    out_host = {n: torch.empty(t.shape, dtype=t.dtype).pin_memory() for n, t in out_like.items() if t is not None}
    pipe = HostPipeline(host_in, dev)

    def e2e_step():
        pipe.run(host_in, out_host, w.causal, w.softmax_scale)

    e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    d2h = sum(t.numel() * t.element_size() for t in out_host.values())

    ms_step = ms_total / args.steps
    stats = torch.tensor([ms_step, e2e_ms, fwd_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    ms_step, e2e_ms, fwd_ms = (float(x) for x in stats.cpu())

    if rank == 0:
        peaks = load_peaks()
        fl = fl_f + fl_b
        value = world * fl / (ms_step * 1e-3) / 1e12
        bwd_kernel_ms = kms.value / max(kn.value, 1)
        ach = fl_b / (bwd_kernel_ms * 1e-3) / 1e12 if kn.value else None
        fwd_kernel_ms = fkms.value / max(fkn.value, 1)
        # algorithmic bytes of one backward call: reads q,k,v,o,dO,factors,lse,delta; writes dq,dk,dv,dq_bias,dk_bias
        nfac = (w.q_bias.numel() + w.k_bias.numel()) if w.q_bias is not None else 0
        bytes_b = 2 * (sh["B"] * sh["H"] * (4 * sh["Sq"] * sh["D"] + 4 * sh["Sk"] * sh["D"]) + 2 * nfac) + \
            8 * sh["B"] * sh["H"] * sh["Sq"]
        t_b = bwd_kernel_ms * 1e-3
        tensor = {"achieved": ach, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                  "frac": (ach / peaks["bf16_tflops"]) if ach else None}
        gbs = bytes_b / t_b / 1e9 if kn.value else None
        hbm = {"achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
               "frac": (gbs / peaks["hbm_gbs"]) if gbs else None}
        # the binding roofline is the one with the larger lower bound on the kernel's time
        hbm_binds = bytes_b / (peaks["hbm_gbs"] * 1e9) > fl_b / (peaks["bf16_tflops"] * 1e12)
        roof = {"bound": "hbm" if hbm_binds else "tensor", "kernel": "bwd_sm100_kernel",
                **(hbm if hbm_binds else tensor), "peak_source": peaks["source"],
                "ms_per_launch": bwd_kernel_ms, "launches_timed": kn.value, "flop_per_launch": fl_b,
                "bytes_per_launch": bytes_b, "other_roofline": tensor if hbm_binds else hbm,
                # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel, from the ncu capture
                # summarised in profiles/bench_alibi_launch_list.md (full-size alibi workload)
                "traffic": NCU_BWD_TRAFFIC_BYTES.get(args.workload)}
        # the reference's own flop convention (benchmark.py: (4D+1) B H S^2 forward, x3 forward+backward, no
        # causal discount), so that numbers can be laid beside its tables
        ref_fl = 3.0 * (4 * sh["D"] + 1) * sh["B"] * sh["H"] * sh["Sq"] * sh["Sk"]
        line = {
            "metric": "fwd+bwd attention TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if w.dtype == torch.bfloat16 else "f16",
            "data": "synthetic",
            "config": {"workload": args.workload, **sizes, "causal": w.causal, "rank": sh["R"],
                       "l2": "flushed between steps (256 MiB write)", "per_gpu_batch": sh["B"],
                       "fwd_ms": fwd_ms, "fwd_tflops": world * fl_f / (fwd_ms * 1e-3) / 1e12,
                       "fwd_kernel_ms": fwd_kernel_ms,
                       "fwd_kernel_tflops": fl_f / (fwd_kernel_ms * 1e-3) / 1e12 if fkn.value else None,
                       "flop_convention": "T*(14D+8R), T = attended (query,key) pairs",
                       "reference_convention_tflops": world * ref_fl / (ms_step * 1e-3) / 1e12},
            "clocks": clocks,
            "e2e": {"value": world * fl / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": int(launches),
            "roofline": roof,
        }
        if not args.no_cpu_baseline and world == 1:
            from oracle import flashbias_oracle as orc
            cores = os.cpu_count() or 1
            torch.set_num_threads(cores)
            cs, what = CPU_SAMPLE[args.workload]
            cw = make_workload(args.workload, **cs)
            csh = cw.shape
            cfl = flops_fwd(csh["B"], csh["H"], csh["Sq"], csh["Sk"], csh["D"], csh["R"], cw.causal) + \
                flops_bwd(csh["B"], csh["H"], csh["Sq"], csh["Sk"], csh["D"], csh["R"], cw.causal)
            f32 = [t.float() for t in (cw.q, cw.k, cw.v, cw.q_bias, cw.k_bias)]
            t0 = time.perf_counter()
            n = 0
            while n < 1 or (time.perf_counter() - t0 < 10.0 and n < 5):
                orc.attention_forward_backward(*f32, None, cw.causal, cw.softmax_scale, cw.do.float())
                n += 1
            cdt = (time.perf_counter() - t0) / n
            line["cpu_baseline"] = {"value": cfl / cdt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                    "sample": f"{what}, {n} pass(es) of {cdt:.2f} s; fp32 naive attention, torch CPU ops"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
