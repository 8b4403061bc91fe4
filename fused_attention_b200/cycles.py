"""SM clock counts of launches of the warp-specialised kernels (a diagnostic, not part of the operator).

The clock-counting build of the library (``python -m fused_attention_b200.build --cycles``, -DFA_CYCLES) makes
CTA 0 of ``fa_fwd_pipelined`` and ``fa_fwd_pair`` record, per launch, the global timer at its entry, after its
wait for the previous kernel of the stream and at its end, and its SM clock count between the last two.  A
kernel's SM clock count does not depend on the clock the power cap allows at the moment, which is what makes
it the figure to compare two versions of a kernel by.

    python -m fused_attention_b200.cycles B R L H [flags]      # e.g. 4 32 2048 128 32

prints the medians over a loop of launches; ``measure`` returns them.

The time-line build (-DFA_CYCLES -DFA_TIMELINE, same build command) also stamps, for the kernel on pairs of
CTAs at head_dim 128, the events of every key step as seen by one softmax warp of each query tile and by the two
warps that issue the MMAs:

    python -m fused_attention_b200.cycles --timeline B R L H   # e.g. --timeline 4 32 2048 128

prints where a key step's clocks go (``timeline`` returns the same as a dict).
"""
from __future__ import annotations

import ctypes
import os
import sys

from . import build


def _load(path: str | None = None) -> ctypes.CDLL:
    path = path or build.CYCLES_LIB
    if not os.path.exists(path):
        raise RuntimeError(f"{path} is missing: python -m fused_attention_b200.build --cycles")
    lib = ctypes.CDLL(path)
    u32, vp, i32 = ctypes.c_uint32, ctypes.c_void_p, ctypes.c_int
    lib.fa_b200_attention_forward.restype = i32
    lib.fa_b200_attention_forward.argtypes = [vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, i32, vp, u32]
    lib.fa_b200_debug_cycles.restype = i32
    lib.fa_b200_debug_cycles.argtypes = [vp]
    return lib


def parse_records(words: list[int]) -> list[dict]:
    """The device buffer is 64 records of four 64-bit words {entry ns, past-wait ns, end ns, SM clocks from
    past-wait to end}, indexed by the launch id modulo 64; unused records are zero."""
    recs = []
    for i in range(0, len(words) - 3, 4):
        entry, ready, end, clocks = words[i:i + 4]
        if entry and ready >= entry and end >= ready:
            recs.append({"entry_ns": entry, "ready_ns": ready, "end_ns": end, "sm_clocks": clocks})
    recs.sort(key=lambda r: r["entry_ns"])
    return recs


def summarise(recs: list[dict]) -> dict:
    """Medians over consecutive launches: SM clocks and busy time of CTA 0, start-to-start period, and the gap
    from CTA 0's end to the next launch's CTA 0 being past its wait."""
    def med(xs):
        xs = sorted(xs)
        return xs[len(xs) // 2] if xs else None
    return {
        "launches": len(recs),
        "sm_clocks": med([r["sm_clocks"] for r in recs]),
        "busy_us": med([(r["end_ns"] - r["ready_ns"]) / 1e3 for r in recs]),
        "period_us": med([(b["ready_ns"] - a["ready_ns"]) / 1e3 for a, b in zip(recs, recs[1:])]),
        "gap_us": med([(b["ready_ns"] - a["end_ns"]) / 1e3 for a, b in zip(recs, recs[1:])]),
    }


def measure(B: int, R: int, L: int, H: int, flags: int = 0, launches: int = 40, device: int = 0) -> dict:
    import torch
    from .workloads import make_inputs

    lib = _load()
    dev = torch.device("cuda", device)
    torch.cuda.set_device(device)
    buf = torch.zeros(256, dtype=torch.int64, device=dev)
    lib.fa_b200_debug_cycles(buf.data_ptr())
    one = 4 * B * L * R * H * 2
    n = max(2, min(24, -(-300 * 2 ** 20 // one)))      # rotate over more than L2
    ins = [tuple(t.to(dev) for t in make_inputs(B, L, R * H, 0.5, 100 + i)) for i in range(n)]
    y = torch.empty_like(ins[0][0])

    def launch(i):
        q, k, v = ins[i % n]
        rc = lib.fa_b200_attention_forward(q.data_ptr(), k.data_ptr(), v.data_ptr(), None, y.data_ptr(), B, L, R * H,
                                           H, 0, device, None, flags)
        if rc != 0:
            raise RuntimeError(f"fa_b200_attention_forward returned {rc}")
    try:
        for i in range(10):
            launch(i)
        torch.cuda.synchronize(dev)
        buf.zero_()
        launches = min(launches, 60)
        for i in range(launches):
            launch(i)
        torch.cuda.synchronize(dev)
        recs = parse_records(buf.cpu().tolist())
    finally:
        lib.fa_b200_debug_cycles(None)
    out = summarise(recs[2:-2] if len(recs) > 8 else recs)
    out.update({"B": B, "R": R, "L": L, "H": H, "flags": flags})
    return out


TIMELINE_WORDS = 9 * 1024      # 256 words of launch records, then 4 roles x 256 key steps x 8 events
_SOFTMAX_EVENTS = ("looks for S", "S there", "S in registers", "first 32 exponentials taken", "P buffer free",
                   "exponentials taken, P stored", "P handed over")


def parse_timeline(words: list[int], lo: int = 20, hi: int = 100) -> dict:
    """Mean durations (SM clocks) over key steps [lo, hi) of CTA 0 from the words the time-line build wrote behind
    the launch records: role 0, 1 = a softmax warp of query tile 0, 1 (events as in _SOFTMAX_EVENTS), role 2 = the
    warp issuing Q K^T (0 top of the step, 1 K there, 2 issues tile 0's, 3 issued, 4 issues tile 1's, 5 issued),
    role 3 = the warp issuing P V (the same with V and P).  A stamp of 0 means "not reached"."""
    def at(role, g, ev):
        return words[256 + (role * 256 + g) * 8 + ev]

    def mean(xs):
        xs = [x for x in xs if x is not None]
        return sum(xs) / len(xs) if xs else None

    def span(role_a, ev_a, role_b, ev_b, dg=0):
        out = []
        for g in range(lo, hi - dg):
            a, b = at(role_a, g, ev_a), at(role_b, g + dg, ev_b)
            if a and b:
                out.append(b - a)
        return mean(out)

    res = {"steps_recorded": sum(1 for g in range(256) if at(2, g, 2)),
           "step_period": span(2, 2, 2, 2, 1)}
    for i in (0, 1):
        res[f"tile{i}"] = {
            "wait_for_S": span(i, 0, i, 1), "S_into_registers_and_first_32_exponentials": span(i, 1, i, 3),
            "wait_for_P_buffer": span(i, 3, i, 4), "other_96_exponentials_and_P_stores": span(i, 4, i, 5),
            "hand_over": span(i, 5, i, 6), "pass": span(i, 1, i, 6),
        }
    res["qk_warp"] = {"wait_for_K": span(2, 0, 2, 1), "wait_for_S_read_by_tile1": span(2, 1, 2, 2),
                      "wait_for_S_read_by_tile0": span(2, 3, 2, 4)}
    res["pv_warp"] = {"wait_for_V": span(3, 0, 3, 1), "wait_for_P0": span(3, 1, 3, 2), "wait_for_P1": span(3, 3, 3, 4)}
    res["S_finished_before_its_tile_looks"] = {
        # Q K^T of tile i issued -> its softmax warp sees S: MMA time + hand-over + how long the warp was still busy
        "tile0_issue_to_seen": span(2, 2, 0, 1), "tile1_issue_to_seen": span(2, 4, 1, 1)}
    return res


def timeline(B: int, R: int, L: int, H: int = 128, device: int = 0) -> dict:
    """One launch of the kernel on pairs of CTAs (forced) after a few warm-up launches; its time line parsed."""
    import torch
    from .workloads import make_inputs
    from ._lib import FLAG_FORCE_PAIR

    lib = _load(build.TIMELINE_LIB)
    dev = torch.device("cuda", device)
    torch.cuda.set_device(device)
    buf = torch.zeros(TIMELINE_WORDS, dtype=torch.int64, device=dev)
    lib.fa_b200_debug_cycles(buf.data_ptr())
    ins = [tuple(t.to(dev) for t in make_inputs(B, L, R * H, 0.5, 100 + i)) for i in range(3)]
    y = torch.empty_like(ins[0][0])
    try:
        for i in range(7):
            if i == 6:
                torch.cuda.synchronize(dev)
                buf.zero_()
            q, k, v = ins[i % 3]
            rc = lib.fa_b200_attention_forward(q.data_ptr(), k.data_ptr(), v.data_ptr(), None, y.data_ptr(), B, L, R * H,
                                               H, 0, device, None, FLAG_FORCE_PAIR)
            if rc != 0:
                raise RuntimeError(f"fa_b200_attention_forward returned {rc}")
        torch.cuda.synchronize(dev)
        words = buf.cpu().tolist()
    finally:
        lib.fa_b200_debug_cycles(None)
    steps = sum(1 for g in range(256) if words[256 + (2 * 256 + g) * 8 + 2])
    return parse_timeline(words, lo=min(20, steps // 4), hi=max(min(100, steps - 4), min(20, steps // 4) + 1))


if __name__ == "__main__":
    args = sys.argv[1:]
    if args and args[0] == "--timeline":
        a = [int(x) for x in args[1:]]
        if len(a) not in (3, 4):
            sys.exit(__doc__)
        import json
        print(json.dumps(timeline(*a), indent=1))
        sys.exit(0)
    a = [int(x) for x in args]
    if len(a) not in (4, 5):
        sys.exit(__doc__)
    print(measure(*a))
