"""SM clock counts of launches of the warp-specialised kernels (a diagnostic, not part of the operator).

The clock-counting build of the library (``python -m fused_attention_b200.build --cycles``, -DFA_CYCLES) makes
CTA 0 of ``fa_fwd_pipelined`` and ``fa_fwd_pair`` record, per launch, the global timer at its entry, after its
wait for the previous kernel of the stream and at its end, and its SM clock count between the last two.  A
kernel's SM clock count does not depend on the clock the power cap allows at the moment, which is what makes
it the figure to compare two versions of a kernel by.

    python -m fused_attention_b200.cycles B R L H [flags]      # e.g. 4 32 2048 128 32

prints the medians over a loop of launches; ``measure`` returns them.
"""
from __future__ import annotations

import ctypes
import os
import sys

from . import build


def _load() -> ctypes.CDLL:
    if not os.path.exists(build.CYCLES_LIB):
        raise RuntimeError(f"{build.CYCLES_LIB} is missing: python -m fused_attention_b200.build --cycles")
    lib = ctypes.CDLL(build.CYCLES_LIB)
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


if __name__ == "__main__":
    a = [int(x) for x in sys.argv[1:]]
    if len(a) not in (4, 5):
        sys.exit(__doc__)
    print(measure(*a))
