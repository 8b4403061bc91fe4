"""Compile the reference's own CUDA kernel into oracle/_ref/libref_fused_attn.so (test infrastructure).

  python oracle/build_ref.py [/path/to/reference]

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


def build(ref_root: str = "/root/reference", force: bool = False) -> str | None:
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
    print(build(sys.argv[1] if len(sys.argv) > 1 else "/root/reference", force="--force" in sys.argv))
