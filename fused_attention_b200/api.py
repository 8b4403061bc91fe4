"""Host-side mirror of the reference operator, on top of the C ABI.

``attention_forward`` has the signature, argument meaning and error behaviour of the reference's
torch binding (``src/fused_attn_extention.cu:15-117``): fp16 CUDA contiguous rank-3 tensors
``[B, L, F]``, ``RuntimeError`` on any violated precondition, a freshly allocated fp16 output.
Differences, all relaxations: ``L`` need not be a multiple of ``chunk_size`` (ragged tails are
masked inside the kernel), the output is allocated on ``queries.device`` (the reference uses the
current device, ``:67-70``), the launch goes to the caller's current stream, and the mask is
applied to every key tile (the reference applies it to the first chunk only,
``include/fused_attn.cuh:732-742``).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib


def _require(cond: bool, what: str) -> None:
    if not cond:
        raise RuntimeError(f"attention_forward: {what}")


def _check_tensor(t: torch.Tensor, name: str) -> None:
    # src/fused_attn_extention.cu:24-43
    _require(isinstance(t, torch.Tensor), f"{name} must be a tensor")
    _require(t.dtype == torch.float16, f"{name} must be float16")
    _require(t.device.type == "cuda", f"{name} must be a CUDA tensor")
    _require(t.is_contiguous(), f"{name} must be contiguous")
    _require(t.dim() == 3, f"{name} must have 3 dimensions")


def attention_forward(head_dim: int, chunk_size: int, queries: torch.Tensor, keys: torch.Tensor,
                      values: torch.Tensor, mask: Optional[torch.Tensor] = None, *,
                      flags: int = _lib.FLAG_DEFAULT) -> torch.Tensor:
    """Fused multi-head attention forward ``softmax(Q K^T / sqrt(head_dim)) V`` on the GPU."""
    lib = _lib.load()  # raises when the CUDA library is missing: no fallback
    _check_tensor(queries, "queries")
    _check_tensor(keys, "keys")
    _check_tensor(values, "values")
    if mask is not None:
        _check_tensor(mask, "mask")
    head_dim, chunk_size = int(head_dim), int(chunk_size)
    # src/fused_attn_extention.cu:45-47
    _require(head_dim > 0 and not (head_dim & (head_dim - 1)) and 16 <= head_dim <= 128,
             "head_dim must be a power of two in [16, 128]")
    _require(chunk_size > 0 and not (chunk_size & (chunk_size - 1)) and 16 <= chunk_size <= 128
             and chunk_size <= 2 * head_dim, "chunk_size must be a power of two in [16, 128] and <= 2*head_dim")
    _require(not (chunk_size == 16 and head_dim == 128), "chunk_size 16 with head_dim 128 is not supported")
    B, L, F = queries.shape
    # :55-64 (the L % chunk_size requirement is lifted)
    _require(tuple(keys.shape) == (B, L, F), "keys must have the shape of queries")
    _require(tuple(values.shape) == (B, L, F), "values must have the shape of queries")
    _require(F % head_dim == 0, "the feature size must be divisible by head_dim")
    _require(B > 0 and L > 0 and F > 0, "empty tensors are not supported")
    _require(keys.device == queries.device and values.device == queries.device,
             "queries, keys and values must be on one device")
    if mask is not None:
        _require(tuple(mask.shape) == (B, L, L), "mask must have shape [B, L, L]")
        _require(mask.device == queries.device, "mask must be on the device of queries")
    out = torch.empty_like(queries)
    dev = queries.device.index if queries.device.index is not None else torch.cuda.current_device()
    stream = torch.cuda.current_stream(queries.device).cuda_stream
    rc = lib.fa_b200_attention_forward(
        queries.data_ptr(), keys.data_ptr(), values.data_ptr(),
        mask.data_ptr() if mask is not None else None, out.data_ptr(),
        B, L, F, head_dim, chunk_size, dev, ctypes.c_void_p(stream), int(flags))
    _lib.check(rc)
    return out


def bind_forward(head_dim: int, chunk_size: int, queries: torch.Tensor, keys: torch.Tensor, values: torch.Tensor,
                 mask: Optional[torch.Tensor] = None, *, out: Optional[torch.Tensor] = None,
                 flags: int = _lib.FLAG_DEFAULT):
    """The same call with its arguments checked and converted once: returns ``(launch, out)`` where ``launch()``
    does nothing but call ``fa_b200_attention_forward`` on the current stream of the tensors' device, writing
    into ``out``.  For loops over fixed tensors (benchmarks, CUDA-graph capture), where the checks and the
    allocation of ``attention_forward`` would cost more than a small problem's kernel."""
    lib = _lib.load()
    probe = attention_forward   # the checks live there; run them once on these tensors
    y = probe(head_dim, chunk_size, queries, keys, values, mask, flags=flags)
    if out is None:
        out = y
    else:
        _check_tensor(out, "out")
        _require(tuple(out.shape) == tuple(queries.shape) and out.device == queries.device, "out must match queries")
    B, L, F = queries.shape
    dev = queries.device.index if queries.device.index is not None else torch.cuda.current_device()
    ptrs = (queries.data_ptr(), keys.data_ptr(), values.data_ptr(), mask.data_ptr() if mask is not None else None,
            out.data_ptr())
    fn, device, H, C, fl = lib.fa_b200_attention_forward, queries.device, int(head_dim), int(chunk_size), int(flags)
    keep = (queries, keys, values, mask, out)   # the tensors live as long as the closure

    def launch() -> None:
        stream = torch.cuda.current_stream(device).cuda_stream
        rc = fn(ptrs[0], ptrs[1], ptrs[2], ptrs[3], ptrs[4], B, L, F, H, C, dev, ctypes.c_void_p(stream), fl)
        if rc != 0:
            _lib.check(rc)
    launch.tensors = keep
    return launch, out


def attention_forward_host(head_dim: int, chunk_size: int, queries: torch.Tensor, keys: torch.Tensor,
                           values: torch.Tensor, mask: Optional[torch.Tensor] = None, *, device: int = 0,
                           out: Optional[torch.Tensor] = None, flags: int = _lib.FLAG_DEFAULT) -> torch.Tensor:
    """Same operator for HOST tensors: copies in, runs on ``device``, copies out, returns when done.

    Goes through ``fa_b200_attention_forward_host``; pinned tensors make the copies asynchronous
    with respect to the host and reach full PCIe speed.
    """
    lib = _lib.load()
    for t, name in ((queries, "queries"), (keys, "keys"), (values, "values")) + (
            ((mask, "mask"),) if mask is not None else ()):
        _require(t.dtype == torch.float16 and t.device.type == "cpu" and t.is_contiguous() and t.dim() == 3,
                 f"{name} must be a contiguous float16 CPU tensor of rank 3")
    B, L, F = queries.shape
    _require(tuple(keys.shape) == (B, L, F) and tuple(values.shape) == (B, L, F), "shape mismatch")
    if mask is not None:
        _require(tuple(mask.shape) == (B, L, L), "mask must have shape [B, L, L]")
    if out is None:
        out = torch.empty_like(queries)
    else:
        _require(out.dtype == torch.float16 and out.device.type == "cpu" and out.is_contiguous()
                 and tuple(out.shape) == (B, L, F), "out must match queries")
    rc = lib.fa_b200_attention_forward_host(
        queries.data_ptr(), keys.data_ptr(), values.data_ptr(),
        mask.data_ptr() if mask is not None else None, out.data_ptr(),
        B, L, F, int(head_dim), int(chunk_size), int(device), int(flags))
    _lib.check(rc)
    return out


def read_status(device: int = 0) -> tuple[int, int]:
    """(first failure code, reporting CTA count) of the device status word; clears it."""
    w = (ctypes.c_uint32 * 2)()
    _lib.check(_lib.load().fa_b200_read_status(int(device), w))
    return int(w[0]), int(w[1])


def query(device: int = 0) -> dict:
    o = (ctypes.c_int32 * 4)()
    _lib.check(_lib.load().fa_b200_query(int(device), o))
    return {"cc_major": o[0], "cc_minor": o[1], "sm_count": o[2], "smem_optin": o[3]}


def select_kernel(B: int, L: int, F: int, head_dim: int, has_mask: bool = False, flags: int = 0) -> str:
    rc = _lib.load().fa_b200_select_kernel(B, L, F, head_dim, int(has_mask), flags)
    if rc < 0:
        _lib.check(rc)
    return {1: "simple", 2: "pipelined", 3: "pipelined on pairs of CTAs"}[rc]


def describe_schedule(B: int, L: int, F: int, head_dim: int, flags: int = 0, sm_count: int = 148) -> dict:
    """How the warp-specialised kernel spreads a call over its CTAs (``fa_b200_describe_schedule``)."""
    o = (ctypes.c_uint32 * 7)()
    _lib.check(_lib.load().fa_b200_describe_schedule(B, L, F, head_dim, int(flags), int(sm_count), o))
    return {"kernel": {1: "simple", 2: "pipelined", 3: "pipelined on pairs of CTAs"}[o[0]], "grid": o[1], "full_rounds": o[2],
            "tail_items": o[3], "tail_steps": o[4], "key_steps": o[5], "tail_grid": o[6]}


def cta_segments(sched: dict, n_items: int, cta: int) -> list[tuple[int, int, int]]:
    """The (work item, first key step, key steps) runs that CTA ``cta`` works through under ``sched``, in
    the kernel's order and with its arithmetic: whole items round-robin, then its share of a divided
    round (at most two runs)."""
    grid, n, T = sched["grid"], sched["key_steps"], sched["tail_steps"]
    if T == 0:
        return [(item, 0, n) for item in range(cta, n_items, grid)]
    segs = [(cta + k * grid, 0, n) for k in range(sched["full_rounds"])]
    tg = sched["tail_grid"]
    a, b = (cta * T // tg, (cta + 1) * T // tg) if cta < tg else (0, 0)
    base = sched["full_rounds"] * grid
    if b > a:
        t0, j0 = divmod(a, n)
        len0 = min(n - j0, b - a)
        segs.append((base + t0, j0, len0))
        if b - a > len0:
            segs.append((base + t0 + 1, 0, b - a - len0))
    return segs
