"""Build the native parts in-tree.

  libfa_b200.so   CUDA kernels + C ABI (torch-free), nvcc, sm_100a only
  fused_attn*.so  the torch extension module ``fused_attn`` (thin C++ binding over the C ABI)

  bin/fa_b200_driver  torch-free C++ program over the C ABI (fill, run, check, time)

Run ``python -m fused_attention_b200.build [--ext] [--driver] [--debug] [--cycles]`` (``--debug`` also builds the
checked library ``lib/libfa_b200_debug.so``, ``--cycles`` the clock-counting ones ``lib/libfa_b200_cycles.so`` and
``lib/libfa_b200_timeline.so``).
Nothing is installed outside the tree.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
EXTDIR = os.path.join(HERE, "ext")
LIB = os.path.join(LIBDIR, "libfa_b200.so")
DEBUG_LIB = os.path.join(LIBDIR, "libfa_b200_debug.so")   # the checked build (-DFA_DEBUG), used by one GPU test
CYCLES_LIB = os.path.join(LIBDIR, "libfa_b200_cycles.so")  # the clock-counting build (-DFA_CYCLES), see cycles.py
TIMELINE_LIB = os.path.join(LIBDIR, "libfa_b200_timeline.so")  # ... with per-step time stamps (-DFA_TIMELINE) as well

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def lib_sources() -> list[str]:
    return [os.path.join(CSRC, f) for f in ("fa_b200.cu", "fa_kernels.cuh", "fa_pair.cuh", "fa_ptx.cuh")] + [
        os.path.join(ROOT, "include", "fa_b200.h")]


def build_lib(force: bool = False, verbose: bool = False, debug: bool = False, cycles: bool = False,
              timeline: bool = False) -> str:
    """Compile csrc/fa_b200.cu into lib/libfa_b200.so (cross-compiles without a GPU).

    ``debug`` builds lib/libfa_b200_debug.so instead, with -DFA_DEBUG: every TMA copy and tensor-memory
    access checks its operands first (see the checked-build section of csrc/fa_ptx.cuh).
    ``cycles`` builds lib/libfa_b200_cycles.so, with -DFA_CYCLES: CTA 0 of the warp-specialised kernels
    records time stamps and its SM clock count per launch (read by cycles.py).
    ``timeline`` builds lib/libfa_b200_timeline.so, with -DFA_CYCLES -DFA_TIMELINE: one warp per role of CTA 0 of
    the kernel on pairs of CTAs also stamps the events of every key step (cycles.py --timeline)."""
    os.makedirs(LIBDIR, exist_ok=True)
    out = DEBUG_LIB if debug else (TIMELINE_LIB if timeline else (CYCLES_LIB if cycles else LIB))
    if not force and not _stale(out, lib_sources()):
        return out
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", os.path.join(ROOT, "include"), "-I", CSRC]
    if debug:
        cmd += ["-DFA_DEBUG"]
    elif timeline:
        cmd += ["-DFA_CYCLES", "-DFA_TIMELINE"]
    elif cycles:
        cmd += ["-DFA_CYCLES"]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", out, os.path.join(CSRC, "fa_b200.cu")]
    subprocess.run(cmd, check=True)
    return out


def ext_path() -> str:
    return os.path.join(EXTDIR, "fused_attn" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_ext(force: bool = False) -> str:
    """Compile csrc/fused_attn_binding.cpp into ext/fused_attn<abi>.so with the host compiler.

    The binding has no device code, so g++ is enough; it links libfa_b200.so by relative rpath.
    """
    import torch
    from torch.utils import cpp_extension as ce

    build_lib()
    os.makedirs(EXTDIR, exist_ok=True)
    src = os.path.join(CSRC, "fused_attn_binding.cpp")
    out = ext_path()
    if not force and not _stale(out, [src, LIB]):
        return out
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_home = ce.CUDA_HOME or "/usr/local/cuda"
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=fused_attn",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    for inc in ce.include_paths() + [os.path.join(cuda_home, "include"), sysconfig.get_paths()["include"],
                                     os.path.join(ROOT, "include")]:
        cmd += ["-isystem" if "torch" in inc or "cuda" in inc else "-I", inc]
    cmd += [src, "-o", out, f"-L{torch_lib}", f"-L{LIBDIR}", "-lfa_b200", "-lc10", "-lc10_cuda", "-ltorch_cpu",
            "-ltorch_cuda", "-ltorch", "-ltorch_python", f"-L{os.path.join(cuda_home, 'lib64')}", "-lcudart",
            "-Wl,-rpath,$ORIGIN/../lib", f"-Wl,-rpath,{torch_lib}"]
    subprocess.run(cmd, check=True)
    return out


def driver_path() -> str:
    return os.path.join(HERE, "bin", "fa_b200_driver")


def build_driver(force: bool = False) -> str:
    """Compile csrc/fa_driver.cu, the torch-free program over the C ABI, into bin/fa_b200_driver."""
    build_lib()
    src = os.path.join(CSRC, "fa_driver.cu")
    out = driver_path()
    os.makedirs(os.path.dirname(out), exist_ok=True)
    if not force and not _stale(out, [src, LIB]):
        return out
    cmd = [_nvcc(), "-O2", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-I", os.path.join(ROOT, "include"),
           "-o", out, src, f"-L{LIBDIR}", "-lfa_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../lib"]
    subprocess.run(cmd, check=True)
    return out


def main(argv: list[str]) -> int:
    force = "--force" in argv
    print(build_lib(force=force, verbose="-v" in argv))
    if "--debug" in argv:
        print(build_lib(force=force, verbose="-v" in argv, debug=True))
    if "--cycles" in argv:
        print(build_lib(force=force, verbose="-v" in argv, cycles=True))
        print(build_lib(force=force, verbose="-v" in argv, timeline=True))
    if "--ext" in argv:
        print(build_ext(force=force))
    if "--driver" in argv:
        print(build_driver(force=force))
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
