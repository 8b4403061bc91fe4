"""ctypes loader for ``libfa_b200.so`` (the C ABI declared in ``include/fa_b200.h``).

There is no fallback: if the shared library has not been built, loading raises and every
operator of this package fails.  Build it with ``python -m fused_attention_b200.build``.
"""
from __future__ import annotations

import ctypes
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libfa_b200.so")

# Symbols that include/fa_b200.h declares; tests check the library exports every one of them.
EXPORTED_SYMBOLS = (
    "fa_b200_attention_forward",
    "fa_b200_attention_forward_host",
    "fa_b200_attention_forward_noalloc",
    "fa_b200_strerror",
    "fa_b200_query",
    "fa_b200_read_status",
    "fa_b200_select_kernel",
    "fa_b200_describe_schedule",
    "fa_b200_selftest_bounded_wait",
    "fa_b200_selftest_debug_checks",
)

# Status codes and flags, mirrored from include/fa_b200.h.
OK = 0
ERR_NULL_POINTER = -1
ERR_HEAD_DIM = -2
ERR_CHUNK = -3
ERR_SHAPE = -4
ERR_ALIGNMENT = -5
ERR_ARCH = -6
ERR_DRIVER = -7
ERR_FLAGS = -8
ERR_DEVICE_TIMEOUT = -9
ERR_TOO_LARGE = -10

FLAG_DEFAULT = 0
FLAG_FORCE_SIMPLE = 1
FLAG_FORCE_PIPELINED = 2
FLAG_SYNC = 4
FLAG_NO_OVERLAP = 8
FLAG_NO_SPLIT = 16
FLAG_FORCE_PAIR = 32
FLAG_NO_PAIR = 64

_lock = threading.Lock()
_lib = None


class LibraryNotBuilt(RuntimeError):
    pass


def load() -> ctypes.CDLL:
    """Return the loaded library, loading it on first use.  Raises if it is missing."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise LibraryNotBuilt(
                f"{LIB_PATH} is missing: build the CUDA library first "
                "(python -m fused_attention_b200.build); there is no CPU fallback"
            )
        lib = ctypes.CDLL(LIB_PATH)
        u32, vp, i32 = ctypes.c_uint32, ctypes.c_void_p, ctypes.c_int
        lib.fa_b200_attention_forward.restype = i32
        lib.fa_b200_attention_forward.argtypes = [vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, i32, vp, u32]
        lib.fa_b200_attention_forward_noalloc.restype = i32
        lib.fa_b200_attention_forward_noalloc.argtypes = [vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, i32, vp, u32]
        lib.fa_b200_attention_forward_host.restype = i32
        lib.fa_b200_attention_forward_host.argtypes = [vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, i32, u32]
        lib.fa_b200_strerror.restype = ctypes.c_char_p
        lib.fa_b200_strerror.argtypes = [i32]
        lib.fa_b200_query.restype = i32
        lib.fa_b200_query.argtypes = [i32, ctypes.POINTER(ctypes.c_int32)]
        lib.fa_b200_read_status.restype = i32
        lib.fa_b200_read_status.argtypes = [i32, ctypes.POINTER(ctypes.c_uint32)]
        lib.fa_b200_selftest_bounded_wait.restype = i32
        lib.fa_b200_selftest_bounded_wait.argtypes = [i32, ctypes.POINTER(ctypes.c_uint32)]
        lib.fa_b200_select_kernel.restype = i32
        lib.fa_b200_select_kernel.argtypes = [u32, u32, u32, u32, i32, u32]
        lib.fa_b200_describe_schedule.restype = i32
        lib.fa_b200_describe_schedule.argtypes = [u32, u32, u32, u32, u32, u32, ctypes.POINTER(ctypes.c_uint32)]
        _lib = lib
        return lib


def strerror(code: int) -> str:
    return load().fa_b200_strerror(int(code)).decode()


def check(code: int) -> None:
    """Raise RuntimeError for a non-zero status, as the reference binding's TORCH_CHECKs do."""
    if code != OK:
        raise RuntimeError(f"fa_b200: {strerror(code)} (status {code})")
