"""The named workloads (shapes and value distributions) and the seeded synthetic input generator.

The shapes are the five configurations the benchmark specification lists, plus the two of the
reference's own benchmark script; no dataset is involved:
entries are i.i.d. Gaussian, drawn on the CPU in fp32 from a seeded ``torch.Generator``, scaled by
sigma and rounded to fp16, in the operator's ``[B, L, R*H]`` layout.  The reference's own tests
draw N(0,1) inputs with seed 179 (``tests/test_fused_attn.py:13-25``); seeds here are 179 + index.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    B: int
    R: int
    L: int
    H: int
    sigma: float
    seed: int

    @property
    def F(self) -> int:
        return self.R * self.H

    @property
    def flops(self) -> float:
        return 4.0 * self.B * self.R * self.L * self.L * self.H

    @property
    def bytes(self) -> float:
        return 4.0 * self.B * self.L * self.F * 2


WORKLOADS = {
    "tiny": Workload("tiny", 1, 4, 256, 64, 1.0, 179),
    "bert_base": Workload("bert_base", 8, 12, 512, 64, 1.0, 180),
    "vit_l16_ragged": Workload("vit_l16_ragged", 64, 16, 197, 64, 1.0, 181),
    "llama7b_prefill": Workload("llama7b_prefill", 4, 32, 2048, 128, 0.5, 182),
    "long_context": Workload("long_context", 1, 32, 16384, 128, 1.0, 183),
    # the shape of the reference's own benchmark script (tests/benchmark_fused_attn.py:9-22; README.md:110-127):
    # L=2048, F=5120, H=128 (R=40), N(0,1) inputs, batch 4 and 16
    "ref_readme_b4": Workload("ref_readme_b4", 4, 40, 2048, 128, 1.0, 184),
    "ref_readme_b16": Workload("ref_readme_b16", 16, 40, 2048, 128, 1.0, 185),
}
HEADLINE = "llama7b_prefill"
# the five configurations of the benchmark specification, in its order
BENCH_WORKLOADS = ("tiny", "bert_base", "vit_l16_ragged", "llama7b_prefill", "long_context")


def make_inputs(B: int, L: int, F: int, sigma: float = 1.0, seed: int = 179, pin: bool = False):
    """Three independent fp16 CPU tensors [B, L, F] with N(0, sigma^2) entries."""
    g = torch.Generator(device="cpu")
    g.manual_seed(int(seed))
    out = []
    for _ in range(3):
        t = (torch.randn(B, L, F, generator=g, dtype=torch.float32) * sigma).to(torch.float16)
        out.append(t.pin_memory() if pin else t)
    return tuple(out)


def workload_inputs(w: Workload, heads: slice | None = None, batches: slice | None = None, pin: bool = False):
    """Inputs of a workload, optionally restricted to a head/batch slice (made contiguous).

    The full tensors are always generated so that a slice holds exactly the values the unsliced
    run sees; results of sharded and unsharded runs are then comparable bit for bit.
    """
    q, k, v = make_inputs(w.B, w.L, w.F, w.sigma, w.seed)
    if heads is not None or batches is not None:
        hs = heads if heads is not None else slice(0, w.R)
        bs = batches if batches is not None else slice(0, w.B)
        cols = slice(hs.start * w.H, hs.stop * w.H)
        q, k, v = (t[bs, :, cols].contiguous() for t in (q, k, v))
    if pin:
        q, k, v = (t.pin_memory() for t in (q, k, v))
    return q, k, v
