#!/usr/bin/env python
"""Benchmark of the fused attention forward on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload NAME] [--scaling strong|weak]

A step is one forward pass of the operator over one batch of seeded synthetic input.  The default
workload is the headline configuration (LLaMA-7B-shaped prefill, B=4 R=32 L=2048 H=128, fp16).
With N > 1 (one process per GPU; start it under torch.distributed.run, or let this script do so)
the job is sharded by head across the ranks with no collective in the data path.  `--scaling weak`
(the default): the job has R*N heads, so every rank holds the workload's own R heads and the work
per GPU is fixed.  `--scaling strong`: the one workload is divided, R/N heads per rank.
Rank 0 prints ONE JSON line.

The line carries the device-resident throughput (`value`), the end-to-end throughput through the
host-buffer entry point with the host<->device copies inside the timed region (`e2e`), the tensor
roofline of the kernel (`roofline`) and the naive attention timed on this box's CPU cores
(`cpu_baseline`).  `--impl reference` times that CPU implementation alone, with the same keys.
"""
from __future__ import annotations

import argparse
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

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu
# captures summarised under profiles/ (fa_fwd_pipelined_llama7b_prefill.md, fa_fwd_pipelined_h64_vit_bert.md).
NCU_TRAFFIC_BYTES = {"llama7b_prefill": 244.3e6,   # 201.4 MB read + 42.6 to 43.1 MB write
                     "vit_l16_ragged": 83.4e6,     # 77.5 MB read + 5.0 to 6.6 MB write (the rest of Y is still in L2)
                     "bert_base": 18.9e6}          # 18.9 MB read, Y still in L2


def measured_peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


# ----------------------------------------------------------------------------- clocks (read only)
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the GPU works (reads only)."""

    def __init__(self, index: int):
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
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
            time.sleep(0.002)

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
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


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
        "config": {"workload": w.name, "B": w.B, "R": w.R, "L": w.L, "H": w.H,
                   "what": "naive PyTorch attention of the reference (tests/naive_implementation.py restated in "
                           "oracle/naive_attention.py) on the host CPU"},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


# ----------------------------------------------------------------------------- GPU arm
def run_ours(args, workload, rank: int, world: int, local_rank: int) -> dict | None:
    import torch
    import torch.distributed as dist
    import fused_attention_b200 as fa
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

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    strong = args.scaling == "strong"
    if not strong or world == 1:
        shard = fa.Shard(0, w.B, 0, w.R)   # weak: the job has R * world heads, R of them here
    else:
        shard = fa.shard_units(w.B, w.R, world, rank)
    my_flops = fa.attention_flops(shard.b1 - shard.b0, shard.h1 - shard.h0, w.L, w.H)
    total_flops = sum_over_ranks(my_flops)
    # weak scaling: rank r holds heads [r*R, (r+1)*R) of the N-times wider job, drawn with its own seed
    import dataclasses
    w_rank = w if (strong or world == 1) else dataclasses.replace(w, seed=w.seed + 1000 * rank)
    hq, hk, hv = workload_inputs(w_rank, heads=slice(shard.h0, shard.h1), batches=slice(shard.b0, shard.b1), pin=True)
    shard_bytes = 4 * hq.numel() * 2
    # Rotate over copies of the inputs so that consecutive steps do not find them in L2.
    nbuf = max(2, math.ceil(4 * L2_BYTES / shard_bytes))
    bufs = [tuple(t.to(dev) for t in (hq, hk, hv)) for _ in range(nbuf)]
    chunk = 128 if w.H == 128 else 64
    kernel = fa.select_kernel(shard.b1 - shard.b0, w.L, (shard.h1 - shard.h0) * w.H, w.H)

    def step(i: int):
        q, k, v = bufs[i % nbuf]
        return fa.attention_forward(w.H, chunk, q, k, v)

    for i in range(max(3, args.warmup)):
        y = step(i)
    barrier()
    status = fa.read_status(local_rank)
    sampler = ClockSampler(local_rank)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.start()
    e0.record()
    for i in range(args.steps):
        y = step(i)
    e1.record()
    while not e1.query():
        time.sleep(0.0005)
    clocks = sampler.stop()
    barrier()
    my_ms_per_launch = e0.elapsed_time(e1) / args.steps
    agg = fa.aggregate_throughput(my_flops * args.steps, e0.elapsed_time(e1) * 1e-3, sum_over_ranks, max_over_ranks)
    ms_per_step = agg["seconds"] * 1e3 / args.steps
    value = agg["tflops"]

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
    e2e_value = total_flops / e2e_s / 1e12 if e2e_steps else None
    h2d = sum_over_ranks(3 * hq.numel() * 2)
    d2h = sum_over_ranks(hq.numel() * 2)
    status2 = fa.read_status(local_rank)

    out = None
    if rank == 0:
        peaks, peak_kind = measured_peaks()
        peak = float(peaks["bf16_tflops"])
        achieved = my_flops / (my_ms_per_launch * 1e-3) / 1e12
        out = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if strong else "weak", "vs_baseline": None,
            "dtype": "fp16", "data": "synthetic",
            "config": {"workload": w.name, "B": w.B, "R": w.R if strong else w.R * world, "L": w.L, "H": w.H,
                       "sigma": w.sigma, "seed": w.seed,
                       "sharding": (f"by head, no collective: {shard.h1 - shard.h0} of {w.R if strong else w.R * world} "
                                    f"heads x {shard.b1 - shard.b0} batch entries per GPU"),
                       "kernel": kernel,
                       "l2": f"{nbuf} rotating copies of the inputs, {nbuf * shard_bytes / 2**20:.0f} MiB working "
                             f"set > 126 MiB L2"},
            "pct_of_peak": {"measured_dense_bf16_burst": 100.0 * value / (peak * world),
                            "measured_dense_bf16_sustained": (100.0 * value / (float(peaks["bf16_tflops_sustained"]) * world)
                                                              if "bf16_tflops_sustained" in peaks else None),
                            "nominal_dense_fp16_2250": 100.0 * value / (2250.0 * world), "peak_source": peak_kind},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES.get(w.name),
                         "peak_source": f"{peak_kind} cuBLAS dense bf16 burst",
                         "algorithmic_flops_per_launch": my_flops, "algorithmic_bytes_per_launch": shard_bytes},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": int(d2h), "steps": e2e_steps, "ms_per_step": e2e_s * 1e3,
                    "api": "fa_b200_attention_forward_host (pinned host buffers, synchronous)",
                    "timer": "host wall clock around synchronous calls, max over ranks"},
            "gpu_launches": args.steps * world,
            "clocks": clocks,
            "device_status": list(status) + list(status2),
        }
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            tf, dt, sample = cpu_naive_attention(w, 12.0, threads)
            out["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                   "sample": sample, "seconds": dt}
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
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
    ap.add_argument("--scaling", choices=["strong", "weak"], default="weak")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer measurement (profiling runs)")
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
