"""Generate tests/golden/*.npz from the REFERENCE's own naive attention.

Needs the reference checkout (read-only) to import tests/naive_implementation.py::attention; run
once where the reference checkout is available:   python tests/golden/make_golden.py <reference checkout>
Each file holds fp16 inputs q, k, v [B, L, F], the head_dim, and y = reference attention of the
inputs upcast to fp32, on the CPU.
"""
from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from fused_attention_b200.workloads import make_inputs  # noqa: E402

# (name, B, R, L, H, sigma, seed)
CASES = []
# the reference's 12 unit-test shapes: B=1, R=2, L=2*chunk (tests/test_fused_attn.py:12-67)
for H, C in ((16, 16), (16, 32), (32, 16), (32, 32), (32, 64), (64, 16), (64, 32), (64, 64), (64, 128),
             (128, 32), (128, 64), (128, 128)):
    CASES.append((f"ref_test_h{H}_c{C}", 1, 2, 2 * C, H, 1.0, 179))
CASES.append(("tiny", 1, 4, 256, 64, 1.0, 179))                    # benchmark configuration 1
CASES.append(("ragged_l197", 2, 2, 197, 64, 1.0, 181))             # ViT-shaped ragged length
CASES.append(("ragged_l300_h128", 1, 2, 300, 128, 0.5, 182))       # three key tiles, last one ragged
CASES.append(("short_l5_h32", 3, 3, 5, 32, 1.0, 183))


def main(ref_root: str) -> None:
    spec = importlib.util.spec_from_file_location(
        "ref_naive", os.path.join(ref_root, "tests", "naive_implementation.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    torch.set_num_threads(1)  # one thread: the summation order does not depend on the machine
    for name, B, R, L, H, sigma, seed in CASES:
        q, k, v = make_inputs(B, L, R * H, sigma, seed)
        y = mod.attention(q.float(), k.float(), v.float(), H)
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), q=q.numpy(), k=k.numpy(), v=v.numpy(),
                 y=y.numpy().astype(np.float32), head_dim=np.int32(H))
        print(name, tuple(q.shape), float(y.abs().max()))


if __name__ == "__main__":
    if len(sys.argv) < 2 and not os.environ.get("FA_REFERENCE_ROOT"):
        sys.exit("usage: python tests/golden/make_golden.py <reference checkout>   (or set FA_REFERENCE_ROOT)")
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ["FA_REFERENCE_ROOT"])
