"""Compile the reference's own CUDA kernel into oracle/_ref/libref_fused_attn.so (test infrastructure).

  python oracle/build_ref.py [/path/to/reference]

Without an argument the checkout is looked for in $FA_REFERENCE_ROOT, then in a directory named
`reference` beside this repository.

The reference is header-only (include/fused_attn.cuh); nvcc compiles oracle/ref_wmma_wrapper.cu
against that header in place.  Nothing is copied from the reference; the output directory is
git-ignored.  Returns quietly when the reference checkout is absent.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "libref_fused_attn.so")


def default_ref_root() -> str:
    env = os.environ.get("FA_REFERENCE_ROOT")
    if env:
        return env
    return os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(ref_root: str | None = None, force: bool = False) -> str | None:
    ref_root = ref_root or default_ref_root()
    header = os.path.join(ref_root, "include", "fused_attn.cuh")
    if not os.path.exists(header):
        return OUT if os.path.exists(OUT) else None
    src = os.path.join(HERE, "ref_wmma_wrapper.cu")
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) > max(os.path.getmtime(src), os.path.getmtime(header)):
        return OUT
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
           "-shared", "-w", "-I", os.path.join(ref_root, "include"), "-o", OUT, src]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    print(build(args[0] if args else None, force="--force" in sys.argv))
