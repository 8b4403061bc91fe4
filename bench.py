#!/usr/bin/env python
"""Benchmark of the fused attention forward on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload NAME] [--scaling strong|weak] [--context]

A step is one forward pass of the operator over one batch of seeded synthetic input.  The default
workload is the headline configuration (LLaMA-7B-shaped prefill, B=4 R=32 L=2048 H=128, fp16).
With N > 1 (one process per GPU; start it under torch.distributed.run, or let this script do so)
the job is sharded by head across the ranks with no collective in the data path.
`--scaling strong` (the default): the ONE workload is divided, R/N heads per rank, which is what
"the headline shape sharded by head across N GPUs" means; the line then also carries, as the
sibling block `weak`, the throughput of the N-times wider job (R heads per rank).
`--scaling weak` makes that wider job the headline of the line instead.
Rank 0 prints ONE JSON line.

The line carries the device-resident throughput (`value`), the end-to-end throughput through the
host-buffer entry point with the host<->device copies inside the timed region (`e2e`), the tensor
roofline of the kernel (`roofline`), a loop of the same launches that lasts two seconds
(`sustained`), the other benchmark configurations (`other_workloads`, one GPU only) and the naive
attention timed on this box's CPU cores (`cpu_baseline`).  `--impl reference` times that CPU
implementation alone, with the same keys.  `--context` (one GPU, outside any timed arm) times the
reference project's own CUDA kernel, when the test comparator has been built, and naive fp16
attention in PyTorch on the same inputs, for the tables that compare with the reference's README.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import math
import os
import socket
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "fused attn fwd TFLOP/s (4BRL^2H) fp16"
L2_BYTES = 126 * 1024 * 1024
L2_POLICY = "inputs rotate over copies that together exceed the 126 MiB L2"

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu captures
# summarised under profiles/.  A figure is only quoted while the kernel source still has the hash the
# capture was taken at; otherwise the line says that the capture is stale.
NCU_TRAFFIC = {
    "llama7b_prefill": {"bytes": 247.9e6, "profile": "profiles/fa_fwd_pair_llama7b_prefill.md",
                        "kernel_sha": "fd38a85980b2"},
    "vit_l16_ragged": {"bytes": 82.8e6, "profile": "profiles/fa_fwd_pipelined_h64_vit_bert.md",
                       "kernel_sha": "fd38a85980b2"},
    "bert_base": {"bytes": 19.0e6, "profile": "profiles/fa_fwd_pipelined_h64_vit_bert.md",
                  "kernel_sha": "fd38a85980b2"},
}


def kernel_sha() -> str:
    h = hashlib.sha256()
    for name in ("fa_kernels.cuh", "fa_pair.cuh", "fa_ptx.cuh"):
        with open(os.path.join(ROOT, "fused_attention_b200", "csrc", name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:12]


def traffic_for(workload_name: str):
    t = NCU_TRAFFIC.get(workload_name)
    if t is None:
        return None, "no ncu capture of this workload"
    if t["kernel_sha"] != kernel_sha():
        return None, f"{t['profile']} was captured on an earlier version of the kernel source; not quoted"
    return t["bytes"], f"{t['profile']} (ncu capture of this kernel source, not measured in this run)"


def measured_peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def workload_config(w) -> dict:
    """The `config` object: the workload and nothing else, identical in both arms."""
    return {"workload": w.name, "B": w.B, "R": w.R, "L": w.L, "H": w.H, "l2": L2_POLICY}


# ----------------------------------------------------------------------------- clocks (read only)
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the GPU works (reads only)."""

    def __init__(self, index: int, period_s: float = 0.0005):
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self.period_s = period_s
        self._stop = threading.Event()
        self._thread = None
        self._h = None
        try:
            import pynvml
            self._nv = pynvml
            pynvml.nvmlInit()
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:  # NVML missing: the line then says so
            self._h = None

    _NAMES = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
        0x80: "hw_power_brake_slowdown",
    }

    def _sample(self):
        nv = self._nv
        self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
        try:
            bits = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
        except Exception:
            bits = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
        for bit, name in self._NAMES.items():
            if bits & bit:
                self.reasons.add(name)

    def _loop(self):
        while not self._stop.is_set():
            try:
                self._sample()
            except Exception:
                return
            time.sleep(self.period_s)

    def start(self):
        if self._h is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self) -> dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["nvml unavailable"]}
        s = sorted(self.samples)
        bins: dict[str, int] = {}
        for x in s:
            key = str(100 * (x // 100))
            bins[key] = bins.get(key, 0) + 1
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s), "sm_mhz_min": s[0], "sm_mhz_bins_of_100": bins}


# ----------------------------------------------------------------------------- CPU arm
def cpu_naive_attention(workload, target_s: float, threads: int):
    """Time the naive attention (the reference's CPU path, restated in oracle/) on a bounded sample.

    The sample is whole (batch, head) problems of the workload at its full sequence length: as many
    heads as one call holds comfortably, repeated until about `target_s` seconds of CPU work have
    run.  Returns (tflops, seconds, sample text).
    """
    import torch
    from fused_attention_b200.workloads import make_inputs
    from oracle.naive_attention import attention as oracle_attention

    torch.set_num_threads(threads)
    w = workload
    flops_per_head = 4.0 * w.L * w.L * w.H
    heads = max(1, min(w.R, (1 << 28) // (w.L * w.L)))     # scores of one call stay under 1 GiB
    q, k, v = make_inputs(1, w.L, heads * w.H, w.sigma, w.seed)
    oracle_attention(q, k, v, w.H)                           # warm-up (thread pool, allocator)
    reps, t0 = 0, time.perf_counter()
    while True:
        oracle_attention(q, k, v, w.H)
        reps += 1
        dt = time.perf_counter() - t0
        if dt >= target_s or reps >= 10000:
            break
    text = (f"{reps} x {heads} (batch,head) problems of {w.name} at full L={w.L}, fp32, "
            f"{dt:.1f} s of CPU work")
    return reps * heads * flops_per_head / dt / 1e12, dt, text


def run_reference(args, workload) -> dict:
    """`--impl reference`: the reference's CPU implementation of the path, all host threads."""
    import torch
    from fused_attention_b200.workloads import make_inputs
    from oracle.naive_attention import attention as oracle_attention

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    w = workload
    flops_per_head = 4.0 * w.L * w.L * w.H
    # size one step so that steps + warm-up stay within about two minutes
    q, k, v = make_inputs(1, w.L, w.H, w.sigma, w.seed)
    oracle_attention(q, k, v, w.H)
    t0 = time.perf_counter()
    oracle_attention(q, k, v, w.H)
    t_one = time.perf_counter() - t0
    budget = 120.0 / max(1, args.steps + args.warmup)
    heads = int(max(1, min(w.R, budget / max(t_one, 1e-6))))
    q, k, v = make_inputs(1, w.L, heads * w.H, w.sigma, w.seed)
    for _ in range(args.warmup):
        oracle_attention(q, k, v, w.H)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle_attention(q, k, v, w.H)
    dt = (time.perf_counter() - t0) / args.steps
    tflops = heads * flops_per_head / dt / 1e12
    sample = f"{heads} of {w.B * w.R} (batch,head) problems of {w.name} at full L={w.L} per step, fp32"
    return {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(w),
        "what": "naive PyTorch attention of the reference (tests/naive_implementation.py restated in "
                "oracle/naive_attention.py) on the host CPU",
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


# ----------------------------------------------------------------------------- GPU arm
def device_copies(torch, tensors, dev, min_bytes: int, max_copies: int = 64):
    """Copies of the inputs on the device, enough of them that one pass over all exceeds `min_bytes`."""
    one = 4 * tensors[0].numel() * 2        # q, k, v and the output
    n = max(2, min(max_copies, math.ceil(min_bytes / one)))
    return [tuple(t.to(dev) for t in tensors) for _ in range(n)], n, one


def time_launches(torch, fa, H, chunk, bufs, steps: int, warmup: int, flags: int = 0):
    """Milliseconds per launch of `steps` back-to-back launches (CUDA events on the launching stream)."""
    n = len(bufs)
    out = torch.empty_like(bufs[0][0])
    calls = [fa.bind_forward(H, chunk, *b, out=out, flags=flags)[0] for b in bufs]   # arguments checked once
    for i in range(warmup):
        calls[i % n]()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for i in range(steps):
        calls[i % n]()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def sustained_loop(torch, fa, H, chunk, bufs, flops_per_launch: float, ms_guess: float, local_rank: int,
                   seconds: float = 2.0, span: int = 50) -> dict:
    """The same launches for about `seconds`, timed in spans of `span` launches, with the SM clock sampled
    all the while: what the kernel sustains once the GPU has been loaded for a while, and how the time per
    launch moves with the clock (time x clock = SM kilo-cycles per launch, which does not depend on it)."""
    n = len(bufs)
    y_out = torch.empty_like(bufs[0][0])
    calls = [fa.bind_forward(H, chunk, *b, out=y_out)[0] for b in bufs]
    spans = max(5, int(math.ceil(seconds / (span * ms_guess * 1e-3))))
    events = [torch.cuda.Event(enable_timing=True) for _ in range(spans + 1)]
    sampler = ClockSampler(local_rank)
    torch.cuda.synchronize()
    sampler.start()
    events[0].record()
    i = 0
    for s in range(spans):
        for _ in range(span):
            calls[i % n]()
            i += 1
        events[s + 1].record()
    while not events[-1].query():
        time.sleep(0.001)
    clocks = sampler.stop()
    torch.cuda.synchronize()
    per = sorted(events[s].elapsed_time(events[s + 1]) / span for s in range(spans))
    # the first tenth of the loop is the transition from a cool GPU: leave it out of the median
    tail = sorted(events[s].elapsed_time(events[s + 1]) / span for s in range(spans // 10, spans))
    med = tail[len(tail) // 2]
    out = {"seconds": sum(per) * span * 1e-3, "launches": spans * span, "span": span,
           "ms_per_launch_median": med, "ms_per_launch_min": per[0], "ms_per_launch_max": per[-1],
           "tflops_median": flops_per_launch / (med * 1e-3) / 1e12,
           "tflops_best_span": flops_per_launch / (per[0] * 1e-3) / 1e12, "clocks": clocks}
    if clocks.get("sm_mhz"):
        out["sm_kcycles_per_launch"] = med * clocks["sm_mhz"]      # ms x MHz = thousands of cycles
    return out


def other_workloads(torch, fa, dev, peaks: dict, skip: str) -> dict:
    """Every other benchmark configuration, one GPU, about fifty launches each, against the roofline
    that binds it (tensor pipe for the long sequences, HBM for the short ones)."""
    from fused_attention_b200.workloads import BENCH_WORKLOADS, WORKLOADS, workload_inputs
    out = {}
    for name in BENCH_WORKLOADS:
        if name == skip:
            continue
        w = WORKLOADS[name]
        bufs, n, one = device_copies(torch, workload_inputs(w), dev, 2 * L2_BYTES)
        chunk = 128 if w.H == 128 else 64
        ms = time_launches(torch, fa, w.H, chunk, bufs, steps=50, warmup=5)
        tflops = w.flops / (ms * 1e-3) / 1e12
        gbs = w.bytes / (ms * 1e-3) / 1e9
        t_tensor = w.flops / (float(peaks["bf16_tflops"]) * 1e12)
        t_hbm = w.bytes / (float(peaks["hbm_gbs"]) * 1e9)
        bound = "tensor" if t_tensor >= t_hbm else "hbm"
        out[name] = {"B": w.B, "R": w.R, "L": w.L, "H": w.H, "ms_per_launch": ms, "tflops": tflops,
                     "algorithmic_gbs": gbs, "bound": bound,
                     "frac_of_bound": max(t_tensor, t_hbm) / (ms * 1e-3),
                     "frac_tensor": tflops / float(peaks["bf16_tflops"]), "frac_hbm": gbs / float(peaks["hbm_gbs"]),
                     "kernel": fa.select_kernel(w.B, w.L, w.F, w.H),
                     "l2": (f"{n} rotating copies, {n * one / 2**20:.0f} MiB" +
                            ("" if n * one > L2_BYTES else " (fits in L2: the figure is an L2-resident one)"))}
        del bufs
        torch.cuda.empty_cache()
    return out


def masked_run(torch, fa, dev, w, peaks: dict, unmasked_ms: float) -> dict:
    """The same workload with an additive causal mask [B, L, L] (0 on and below the diagonal, -inf above), one
    GPU: the mask costs B*L*L*2 bytes of reads on top of Q, K, V, Y, and no work is skipped (the operator's mask
    is data, not a causal flag), so the FLOP count is the unmasked one."""
    host = __import__("fused_attention_b200.workloads", fromlist=["workload_inputs"]).workload_inputs(w)
    bufs, n, one = device_copies(torch, host, dev, 2 * L2_BYTES, max_copies=8)
    mask = torch.triu(torch.full((w.L, w.L), float("-inf"), device=dev, dtype=torch.float16), diagonal=1)
    mask = mask.unsqueeze(0).expand(w.B, w.L, w.L).contiguous()
    chunk = 128 if w.H == 128 else 64
    y_out = torch.empty_like(bufs[0][0])
    with_mask = [fa.bind_forward(w.H, chunk, *b, mask, out=y_out)[0] for b in bufs]
    without = [fa.bind_forward(w.H, chunk, *b, out=y_out)[0] for b in bufs]
    steps = 50

    def timed(calls):
        for i in range(3):
            calls[i % n]()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for i in range(steps):
            calls[i % n]()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps
    # the unmasked launches are timed again here, before and after the masked ones, so that the ratio compares
    # runs in the same thermal state (this block runs after the two-second loop has warmed the GPU up)
    ms_plain_before = timed(without)
    ms = timed(with_mask)
    ms_plain_after = timed(without)
    ms_plain = 0.5 * (ms_plain_before + ms_plain_after)
    mask_bytes = w.B * w.L * w.L * 2
    t_tensor = w.flops / (float(peaks["bf16_tflops"]) * 1e12)
    t_hbm = (w.bytes + mask_bytes) / (float(peaks["hbm_gbs"]) * 1e9)
    return {"mask": "causal, additive fp16 [B, L, L]", "ms_per_launch": ms, "tflops": w.flops / (ms * 1e-3) / 1e12,
            "algorithmic_bytes": w.bytes + mask_bytes, "algorithmic_gbs": (w.bytes + mask_bytes) / (ms * 1e-3) / 1e9,
            "bound": "tensor" if t_tensor >= t_hbm else "hbm", "frac_of_bound": max(t_tensor, t_hbm) / (ms * 1e-3),
            "unmasked_ms_per_launch_before_and_after": [ms_plain_before, ms_plain_after],
            "time_over_unmasked": ms / ms_plain, "time_over_the_timed_region": ms / unmasked_ms,
            "kernel": fa.select_kernel(w.B, w.L, w.F, w.H, has_mask=True)}


def run_ours(args, workload, rank: int, world: int, local_rank: int) -> dict | None:
    import dataclasses

    import torch
    import torch.distributed as dist
    import fused_attention_b200 as fa
    from fused_attention_b200 import _lib
    from fused_attention_b200.workloads import workload_inputs

    w = workload
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce(x: float, op) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=op)
        return float(t.item())

    def max_over_ranks(x):
        return reduce(x, dist.ReduceOp.MAX if world > 1 else None)

    def sum_over_ranks(x):
        return reduce(x, dist.ReduceOp.SUM if world > 1 else None)

    chunk = 128 if w.H == 128 else 64
    launches = 0

    def timed_job(strong: bool, steps: int, warmup: int, sample_clocks: bool):
        """K launches of this rank's part of the job (the workload divided by head, or, weak, the
        workload itself as this rank's slice of an N-times wider job); returns the aggregate."""
        nonlocal launches
        if strong and world > 1:
            shard = fa.shard_units(w.B, w.R, world, rank)
            w_rank = w
        else:
            shard = fa.Shard(0, w.B, 0, w.R)
            # weak: rank r holds heads [r*R, (r+1)*R) of the wider job, drawn with its own seed
            w_rank = w if world == 1 else dataclasses.replace(w, seed=w.seed + 1000 * rank)
        my_flops = fa.attention_flops(shard.b1 - shard.b0, shard.h1 - shard.h0, w.L, w.H)
        host = workload_inputs(w_rank, heads=slice(shard.h0, shard.h1), batches=slice(shard.b0, shard.b1), pin=True)
        bufs, nbuf, one = device_copies(torch, host, dev, 4 * L2_BYTES)
        # one pass of the hot path = one call of fa_b200_attention_forward; the Python-side checks and the
        # allocation of the output are done once, outside the timed region (a shard's launch at N = 8 is 30 us)
        y_out = torch.empty_like(bufs[0][0])
        calls = [fa.bind_forward(w.H, chunk, *b, out=y_out)[0] for b in bufs]
        for i in range(warmup):
            calls[i % nbuf]()
        barrier()
        sampler = ClockSampler(local_rank) if sample_clocks else None
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        if sampler:
            sampler.start()
        e0.record()
        for i in range(steps):
            calls[i % nbuf]()
        e1.record()
        while not e1.query():
            time.sleep(0.0002)
        clocks = sampler.stop() if sampler else None
        barrier()
        launches += steps
        my_ms = e0.elapsed_time(e1)
        agg = fa.aggregate_throughput(my_flops * steps, my_ms * 1e-3, sum_over_ranks, max_over_ranks)
        return {"shard": shard, "host": host, "bufs": bufs, "nbuf": nbuf, "bytes": one, "my_flops": my_flops,
                "my_ms_per_launch": my_ms / steps, "ms_per_step": agg["seconds"] * 1e3 / steps,
                "value": agg["tflops"], "total_flops_per_step": agg["total_flops"] / steps, "clocks": clocks}

    strong = args.scaling == "strong"
    warmup = max(3, args.warmup)
    fa.read_status(local_rank)
    main = timed_job(strong, args.steps, warmup, sample_clocks=True)
    status = fa.read_status(local_rank)
    shard, bufs, nbuf = main["shard"], main["bufs"], main["nbuf"]
    hq, hk, hv = main["host"]
    kernel = fa.select_kernel(shard.b1 - shard.b0, w.L, (shard.h1 - shard.h0) * w.H, w.H)

    # Outside the timed region: this rank's shard of Y against the same heads of the undivided job
    # computed on this GPU.  NO_SPLIT keeps every (batch, head) on the schedule it has in the undivided
    # job, for which the shard must reproduce its bits; the default schedule may cut the key axis of some
    # work items differently in the two jobs, which moves the result by fp32 rounding only.
    shard_check = None
    if world > 1 and strong:
        full = tuple(t.to(dev) for t in workload_inputs(w))
        cols = slice(shard.h0 * w.H, shard.h1 * w.H)
        rows = slice(shard.b0, shard.b1)
        y_full = fa.attention_forward(w.H, chunk, *full, flags=_lib.FLAG_NO_SPLIT)[rows, :, cols]
        y_mine = fa.attention_forward(w.H, chunk, *bufs[0], flags=_lib.FLAG_NO_SPLIT)
        y_default = fa.attention_forward(w.H, chunk, *bufs[0])
        torch.cuda.synchronize()
        equal = float(torch.equal(y_mine, y_full))
        diff = float((y_default.float() - y_full.float()).abs().max())
        shard_check = {"bit_equal_to_the_undivided_job_all_ranks": bool(reduce(equal, dist.ReduceOp.MIN) == 1.0),
                       "default_schedule_max_abs_diff": max_over_ranks(diff)}
        del full, y_full, y_mine, y_default
        torch.cuda.empty_cache()

    sustained = None
    if not args.no_sustained:
        sustained = sustained_loop(torch, fa, w.H, chunk, bufs, main["my_flops"], main["my_ms_per_launch"], local_rank)
        launches += sustained["launches"]
        sustained["tflops_median_all_gpus"] = (main["total_flops_per_step"] /
                                               (max_over_ranks(sustained["ms_per_launch_median"]) * 1e-3) / 1e12)

    # end to end: host buffers in, host buffer out, through the host entry point of the C ABI
    hy = torch.empty_like(hq).pin_memory()
    e2e_steps = 0 if args.no_e2e else max(1, min(args.steps, 10))
    for _ in range(2 if e2e_steps else 0):
        fa.attention_forward_host(w.H, chunk, hq, hk, hv, device=local_rank, out=hy)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        fa.attention_forward_host(w.H, chunk, hq, hk, hv, device=local_rank, out=hy)
    e2e_s = max_over_ranks((time.perf_counter() - t0) / max(1, e2e_steps))
    barrier()
    e2e_value = main["total_flops_per_step"] / e2e_s / 1e12 if e2e_steps else None
    h2d = sum_over_ranks(3 * hq.numel() * 2)
    d2h = sum_over_ranks(hq.numel() * 2)
    status2 = fa.read_status(local_rank)
    del bufs, main["bufs"]
    torch.cuda.empty_cache()

    other_scaling = None
    if world > 1 and not args.no_other_scaling:
        o = timed_job(not strong, args.steps, warmup, sample_clocks=False)
        other_scaling = {"scaling": "weak" if strong else "strong", "value": o["value"], "unit": "TFLOP/s",
                         "ms_per_step": o["ms_per_step"],
                         "R_of_the_job": w.R * world if strong else w.R,
                         "heads_per_gpu": o["shard"].h1 - o["shard"].h0}
        del o
        torch.cuda.empty_cache()

    out = None
    peaks, peak_kind = measured_peaks()
    others = masked = None
    if rank == 0 and world == 1 and not args.no_other_workloads:
        others = other_workloads(torch, fa, dev, peaks, skip=w.name)
        if w.B * w.L * w.L * 2 <= 4 << 30:
            masked = masked_run(torch, fa, dev, w, peaks, main["my_ms_per_launch"])
    if rank == 0:
        peak = float(peaks["bf16_tflops"])
        peak_sus = float(peaks.get("bf16_tflops_sustained", 0.0)) or None
        value = main["value"]
        achieved = main["my_flops"] / (main["my_ms_per_launch"] * 1e-3) / 1e12
        traffic, traffic_source = traffic_for(w.name) if world == 1 else (None, "captures are of the one-GPU job")
        out = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": main["ms_per_step"], "higher_is_better": True,
            "scaling": "strong" if strong else "weak", "vs_baseline": None,
            "dtype": "fp16", "data": "synthetic",
            "config": workload_config(w) if (strong or world == 1) else dict(workload_config(w), R=w.R * world),
            "inputs": {"sigma": w.sigma, "seed": w.seed, "distribution": "i.i.d. Gaussian, fp16"},
            "sharding": (f"by head, no collective: {shard.h1 - shard.h0} of {w.R if strong else w.R * world} "
                         f"heads x {shard.b1 - shard.b0} batch entries per GPU"),
            "kernel": kernel,
            "l2": f"{nbuf} rotating copies of the inputs, {nbuf * main['bytes'] / 2**20:.0f} MiB working set > 126 MiB L2",
            "pct_of_peak": {"measured_dense_bf16_burst": 100.0 * value / (peak * world),
                            "measured_dense_bf16_sustained": 100.0 * value / (peak_sus * world) if peak_sus else None,
                            "nominal_dense_fp16_2250": 100.0 * value / (2250.0 * world), "peak_source": peak_kind},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak, "traffic": traffic, "traffic_source": traffic_source,
                         "peak_source": f"{peak_kind} cuBLAS dense bf16 burst",
                         "algorithmic_flops_per_launch": main["my_flops"],
                         "algorithmic_bytes_per_launch": main["bytes"]},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": int(d2h), "steps": e2e_steps, "ms_per_step": e2e_s * 1e3,
                    "api": "fa_b200_attention_forward_host (pinned host buffers, synchronous)",
                    "timer": "host wall clock around synchronous calls, max over ranks"},
            "gpu_launches": args.steps * world,
            "gpu_launches_whole_run_this_rank": launches,
            "clocks": main["clocks"],
            "device_status": list(status) + list(status2),
        }
        if sustained is not None:
            sustained["frac_sustained"] = (sustained["tflops_median"] / peak_sus) if peak_sus else None
            sustained["peak_source"] = f"{peak_kind} cuBLAS dense bf16, seconds-long loop"
            out["sustained"] = sustained
        if shard_check is not None:
            out["shard_check"] = shard_check
        if other_scaling is not None:
            out[other_scaling["scaling"]] = other_scaling
        if others is not None:
            out["other_workloads"] = others
        if masked is not None:
            out["masked"] = masked
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            tf, dt, sample = cpu_naive_attention(w, 12.0, threads)
            out["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                   "sample": sample, "seconds": dt}
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return out


# ----------------------------------------------------------------------------- context (comparators)
def run_context(args, workload) -> dict:
    """One GPU, no bench arm: this library, the reference project's own CUDA kernel (the test comparator
    under oracle/_ref, when it has been built) and naive fp16 attention in PyTorch on the same inputs,
    each timed with CUDA events over a loop of launches."""
    import ctypes

    import torch
    import fused_attention_b200 as fa
    from fused_attention_b200.workloads import workload_inputs

    w = workload
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    bufs, nbuf, one = device_copies(torch, workload_inputs(w), dev, 2 * L2_BYTES, max_copies=8)
    chunk = 128 if w.H == 128 else 64
    steps = max(5, args.steps)
    out = {"context": True, "workload": workload_config(w), "steps": steps,
           "l2": f"{nbuf} rotating copies, {nbuf * one / 2**20:.0f} MiB"}

    def timed(fn):
        for i in range(3):
            fn(i)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        return {"ms_per_call": ms, "tflops": w.flops / (ms * 1e-3) / 1e12}

    out["this_library"] = timed(lambda i: fa.attention_forward(w.H, chunk, *bufs[i % nbuf]))

    def naive(i):
        q, k, v = (t.view(w.B, w.L, w.R, w.H).transpose(1, 2) for t in bufs[i % nbuf])
        return (torch.softmax(q @ k.mT / w.H ** 0.5, -1) @ v).transpose(1, 2).contiguous().view(w.B, w.L, w.F)
    try:
        out["naive_pytorch_fp16"] = timed(naive)
        out["naive_pytorch_fp16"]["scores_mib"] = w.B * w.R * w.L * w.L * 2 / 2**20
    except torch.cuda.OutOfMemoryError:
        out["naive_pytorch_fp16"] = {"unavailable": "the L x L scores do not fit"}

    ref_so = os.path.join(ROOT, "oracle", "_ref", "libref_fused_attn.so")
    if os.path.exists(ref_so) and w.L % chunk == 0:
        lib = ctypes.CDLL(ref_so)
        lib.ref_wmma_attention_forward.restype = ctypes.c_int
        lib.ref_wmma_attention_forward.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_uint32] * 5
        y = torch.empty_like(bufs[0][0])

        def ref(i):
            q, k, v = bufs[i % nbuf]
            lib.ref_wmma_attention_forward(q.data_ptr(), k.data_ptr(), v.data_ptr(), None, y.data_ptr(),
                                           w.B, w.L, w.F, w.H, chunk)
        out["reference_wmma_kernel"] = dict(timed(ref), chunk_size=chunk,
                                            note="the reference's kernel compiled for sm_100a from its own header; "
                                                 "its launcher synchronises the device after every call")
    else:
        out["reference_wmma_kernel"] = {"unavailable": "oracle/_ref is not built, or L is not a multiple of the chunk"}
    return out


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", default=None)
    ap.add_argument("--scaling", choices=["strong", "weak"], default="strong")
    ap.add_argument("--context", action="store_true", help="time the comparators on one GPU instead of a bench arm")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer measurement (profiling runs)")
    ap.add_argument("--no-sustained", action="store_true", help="skip the two-second loop (profiling runs)")
    ap.add_argument("--no-other-workloads", action="store_true", help="skip the other configurations (profiling runs)")
    ap.add_argument("--no-other-scaling", action="store_true", help="N > 1: skip the sibling weak (or strong) job")
    args = ap.parse_args()

    from fused_attention_b200.workloads import HEADLINE, WORKLOADS
    workload = WORKLOADS[args.workload or HEADLINE]

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank == 0:  # the other ranks have nothing to do
            print(json.dumps(run_reference(args, workload)), flush=True)
        return 0
    if args.context:
        if rank == 0:
            print(json.dumps(run_context(args, workload)), flush=True)
        return 0

    if args.gpus > 1 and world == 1:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(free_port()), os.path.abspath(__file__),
               *sys.argv[1:]]
        return subprocess.call(cmd)

    out = run_ours(args, workload, rank, world, local_rank)
    if rank == 0 and out is not None:
        print(json.dumps(out), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
