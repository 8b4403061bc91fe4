"""Per-role time line of one CTA of the pipelined kernel, or its SM clock count.

    python -m fused_attention_b200.trace [--workload NAME] [--cta N] [--dump STEPS]
    python -m fused_attention_b200.trace --cycles [--workload NAME]

Builds ``lib/libfa_b200_trace.so`` from the same sources with ``-DFA_TRACE`` (the normal library has
no tracing code), runs the workload once with one CTA recording ``clock64`` at its hand-over points,
and prints, in SM clocks: the length of a key step, how long the MMA warp spends issuing each group of
MMAs and waiting for each P, and how long a softmax warp spends on each part of its step.  This is a
diagnostic for kernel work; it is not used by the operator, the tests or the benchmark.

``--cycles`` builds ``lib/libfa_b200_cycles.so`` with ``-DFA_CYCLES`` instead: the kernel is the normal one
plus two clock reads in CTA 0 (start and end of its work).  The count does not depend on the clock the
GPU happens to run at, which the launch time under the power cap does, so it is the figure to compare
two versions of the kernel by; the recording code of the time line costs a few per cent itself.
"""
from __future__ import annotations

import argparse
import ctypes
import os
import subprocess
import sys

from . import build as _build

TRACE_LIB = os.path.join(_build.LIBDIR, "libfa_b200_trace.so")
CYCLES_LIB = os.path.join(_build.LIBDIR, "libfa_b200_cycles.so")
MMA_TAGS = {1: "V and next K landed", 2: "P0 ready", 8: "PV0 issued", 4: "next QK0 issued",
            5: "P1 ready", 10: "PV1 issued", 7: "next QK1 issued",
            11: "S buffer free for tile 0", 12: "S buffer free for tile 1"}
SM_TAGS = {1: "S ready", 2: "S in registers", 5: "exponentials issued", 4: "P signalled"}


def build_trace_lib(force: bool = False, cycles_only: bool = False) -> str:
    srcs = _build.lib_sources()
    out = CYCLES_LIB if cycles_only else TRACE_LIB
    if not force and os.path.exists(out) and all(os.path.getmtime(s) < os.path.getmtime(out) for s in srcs):
        return out
    os.makedirs(_build.LIBDIR, exist_ok=True)
    cmd = [_build._nvcc(), *_build.NVCC_FLAGS, "-DFA_CYCLES" if cycles_only else "-DFA_TRACE", "-I",
           os.path.join(_build.ROOT, "include"), "-I", _build.CSRC, "-o", out, os.path.join(_build.CSRC, "fa_b200.cu")]
    subprocess.run(cmd, check=True)
    return out


def _mean(xs):
    xs = list(xs)
    return sum(xs) / len(xs) if xs else float("nan")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--workload", default=None)
    ap.add_argument("--cta", type=int, default=20, help="which CTA records (block index)")
    ap.add_argument("--cycles", action="store_true", help="SM clocks of CTA 0 per launch instead of the time line")
    ap.add_argument("--dump-from", type=int, default=-1, metavar="STEP",
                    help="first key step of the dump (default: the middle of the record); an item of the headline "
                         "workload has 16 key steps, so 14 shows an item boundary")
    ap.add_argument("--dump", type=int, default=0, metavar="N",
                    help="also print the merged time line of all roles over N key steps from the middle of the record")
    args = ap.parse_args(argv)

    import torch
    from .workloads import HEADLINE, WORKLOADS, workload_inputs

    w = WORKLOADS[args.workload or HEADLINE]
    lib = ctypes.CDLL(build_trace_lib(cycles_only=args.cycles))
    u32, vp, i32 = ctypes.c_uint32, ctypes.c_void_p, ctypes.c_int
    lib.fa_b200_attention_forward.restype = i32
    lib.fa_b200_attention_forward.argtypes = [vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, i32, vp, u32]
    lib.fa_b200_trace_setup.argtypes = [vp, u32]
    q, k, v = (t.cuda() for t in workload_inputs(w))
    y = torch.empty_like(q)
    buf = torch.zeros(8 * 512, dtype=torch.int64, device="cuda")

    def run():
        rc = lib.fa_b200_attention_forward(q.data_ptr(), k.data_ptr(), v.data_ptr(), None, y.data_ptr(),
                                           w.B, w.L, w.F, w.H, 0, 0, None, 2)   # 2 = pipelined kernel
        if rc != 0:
            raise RuntimeError(f"status {rc}")

    lib.fa_b200_trace_setup(None, 0)
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    if args.cycles:
        lib.fa_b200_trace_setup(buf.data_ptr(), 0xFFFFFFFF)   # no CTA records a time line; CTA 0 stamps start and end
        counts = []
        for _ in range(11):
            run()
            torch.cuda.synchronize()
            t = buf.cpu()
            counts.append(int(t[7 * 512 + 1] - t[7 * 512]))
        lib.fa_b200_trace_setup(None, 0)
        cyc = sorted(counts)[len(counts) // 2]
        n = (w.L + 127) // 128
        items = ((w.L + 255) // 256) * w.R * w.B
        sms = torch.cuda.get_device_properties(0).multi_processor_count
        steps = -(-items // min(sms, items)) * n           # key steps of CTA 0
        mma_clk = steps * 2 * 2 * (128 * 128 * w.H * 2) / 8192   # two tiles x two products, 8192 FLOP per clock and SM
        print(f"workload {w.name}: {cyc} SM clocks per launch in CTA 0 (median of {len(counts)}), {steps} key steps, "
              f"{cyc / steps:.0f} clocks per key step; the MMAs alone need {mma_clk / steps:.0f}: tensor pipe busy {100 * mma_clk / cyc:.1f} %")
        return 0
    lib.fa_b200_trace_setup(buf.data_ptr(), args.cta)
    run()
    torch.cuda.synchronize()
    lib.fa_b200_trace_setup(None, 0)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(20):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 20
    print(f"workload {w.name}: {ms * 1e3:.1f} us per launch, {w.flops / ms / 1e9:.1f} TFLOP/s (trace build)")

    t = buf.cpu().view(8, 512)
    slots = {0: "mma", 1: "softmax0", 2: "softmax1", 3: "mma_pv"}
    ev = {name: [(x >> 8, x & 255) for x in t[s].tolist() if x] for s, name in slots.items()}
    n = max(1, (w.L + 127) // 128)
    # where P has TMEM columns of its own a second warp issues the P V (slot 3); its stamps are read
    # together with those of the first
    mma = sorted(ev["mma"] + ev.pop("mma_pv"))
    ev["mma"] = mma
    # one stamp per key step: the P V of tile 1 issued
    ends = [c for c, g in mma if g == 10]
    periods = [b - a for a, b in zip(ends, ends[1:])]
    if not periods:
        print("no key steps recorded (does the chosen CTA have work?); events per role:",
              {name: len(e) for name, e in ev.items()}, "MMA tags:", sorted({g for _, g in mma}))
        return 1
    steady = sorted(periods)[: max(1, len(periods) * 3 // 4)]          # drop the item-boundary steps
    print(f"key steps per item: {n}; clocks per key step: median of the steady ones {steady[len(steady) // 2]}, "
          f"all {periods[:24]}")
    seg = {}
    for (c0, g0), (c1, g1) in zip(mma, mma[1:]):
        seg.setdefault((g0, g1), []).append(c1 - c0)
    print("MMA warp, mean clocks from one point to the next:")
    for (g0, g1), vals in seg.items():
        if len(vals) >= 4:
            print(f"  {MMA_TAGS.get(g0, g0):>22} -> {MMA_TAGS.get(g1, g1):<22} {_mean(vals):7.0f}")
    for name in ("softmax0", "softmax1"):
        e = ev[name]
        seg = {}
        for (c0, g0), (c1, g1) in zip(e, e[1:]):
            seg.setdefault((g0, g1), []).append(c1 - c0)
        print(f"{name} (row 0's thread), mean clocks:")
        for (g0, g1), vals in seg.items():
            if len(vals) >= 4:
                print(f"  {SM_TAGS.get(g0, g0):>22} -> {SM_TAGS.get(g1, g1):<22} {_mean(vals):7.0f}")
    if args.dump > 0 and len(ends) > args.dump + 4:
        mid = args.dump_from if 0 <= args.dump_from < len(ends) - args.dump else len(ends) // 2
        lo, hi = ends[mid], ends[mid + args.dump]
        merged = sorted((c, name, g) for name, e in ev.items() for c, g in e if lo <= c <= hi)
        print(f"merged time line of {args.dump} key steps (clocks from the first event):")
        for c, name, g in merged:
            tags = MMA_TAGS if name == "mma" else SM_TAGS
            col = {"mma": 0, "softmax0": 1, "softmax1": 2}[name]
            print(f"  {c - lo:7d}  " + " " * (30 * col) + f"{name}: {tags.get(g, g)}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
