"""B200 (sm_100a) fused multi-head attention forward: a drop-in for the operator of
kst179/fused-attention (``fused_attn.attention_forward``).

Public surface:
  attention_forward(head_dim, chunk_size, queries, keys, values, mask=None)   CUDA tensors
  attention_forward_host(...)                                                  host tensors
  bind_forward(...) -> (launch, out)                                           the same call, checked once, for loops
  shard_units / slice_tensor                                                   multi-GPU slicing
The compute path is the CUDA library ``lib/libfa_b200.so`` behind the C ABI of
``include/fa_b200.h``; there is no CPU path.
"""
from . import _lib
from .api import (attention_forward, attention_forward_host, bind_forward, cta_segments, describe_schedule, query, read_status,
                  select_kernel)
from .sharding import (Shard, aggregate_throughput, attention_bytes, attention_flops, shard_units,
                       slice_tensor)

__all__ = [
    "attention_forward", "attention_forward_host", "bind_forward", "query", "read_status", "select_kernel",
    "describe_schedule", "cta_segments",
    "Shard", "shard_units", "slice_tensor", "attention_flops", "attention_bytes", "aggregate_throughput",
    "_lib",
]
