"""Partition of the (batch x head) units of one attention call across the GPUs of a box.

Heads and batches are independent problems (the reference maps them to independent grid axes,
``include/fused_attn.cuh:681-683,883``), so every rank computes its slice with no exchange.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Shard:
    """What one rank computes: batches [b0, b1) x heads [h0, h1)."""
    b0: int
    b1: int
    h0: int
    h1: int

    @property
    def units(self) -> int:
        return (self.b1 - self.b0) * (self.h1 - self.h0)


def shard_units(B: int, R: int, world: int, rank: int) -> Shard:
    """Slice for ``rank`` of ``world``.

    Heads are split when ``R % world == 0`` (every rank then holds a ``[B, L, (R/world)*H]``
    tensor), else batches when ``B % world == 0``, else heads unevenly (the first ``R % world``
    ranks take one head more; a rank may get none when ``world > R``).
    """
    if world < 1 or not (0 <= rank < world):
        raise ValueError("need 0 <= rank < world")
    if B < 1 or R < 1:
        raise ValueError("B and R must be positive")
    if R % world == 0:
        per = R // world
        return Shard(0, B, rank * per, (rank + 1) * per)
    if B % world == 0:
        per = B // world
        return Shard(rank * per, (rank + 1) * per, 0, R)
    base, extra = divmod(R, world)
    h0 = rank * base + min(rank, extra)
    h1 = h0 + base + (1 if rank < extra else 0)
    return Shard(0, B, h0, h1)


def slice_tensor(t, shard: Shard, head_dim: int):
    """The ``[b1-b0, L, (h1-h0)*H]`` slice of a ``[B, L, R*H]`` tensor (made contiguous)."""
    return t[shard.b0:shard.b1, :, shard.h0 * head_dim:shard.h1 * head_dim].contiguous()


def attention_flops(B: int, R: int, L: int, H: int) -> float:
    """FLOPs of the two contractions: 4 * B * R * L^2 * H (softmax not counted)."""
    return 4.0 * B * R * L * L * H


def attention_bytes(B: int, R: int, L: int, H: int) -> float:
    """Compulsory global-memory bytes: read Q, K, V once, write Y once, fp16."""
    return 4.0 * B * L * R * H * 2


def aggregate_throughput(my_flops: float, my_seconds: float, all_reduce_sum, all_reduce_max) -> dict:
    """Whole-job throughput of a sharded run: total FLOPs of all ranks over the slowest rank's time.

    `all_reduce_sum` / `all_reduce_max` take a float and return the reduction over ranks (identity
    functions for one rank); with torch.distributed they are all_reduce calls on the NCCL (GPU) or
    gloo (CPU tests) backend.  No other exchange happens: the data path has no collective.
    """
    total_flops = all_reduce_sum(float(my_flops))
    seconds = all_reduce_max(float(my_seconds))
    return {"total_flops": total_flops, "seconds": seconds,
            "tflops": total_flops / seconds / 1e12 if seconds > 0 else float("inf")}
