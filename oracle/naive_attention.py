"""CPU oracle for the fused attention forward.  TEST INFRASTRUCTURE, not product code: only
tests/, the smoke check and the benchmark's CPU-baseline leg may import it.

It restates the reference's naive PyTorch attention, tests/naive_implementation.py:4-17:
split the feature axis into heads (:8-10), scores = Q K^T / sqrt(head_dim) (:12), softmax over the
key axis (:13), scores V (:14), heads merged back into the feature axis (:16).  The reference's
arithmetic lives in PyTorch itself (batched matmul and torch.softmax; the reference pins no torch
version), so this restatement uses the same torch primitives in the same order, but walks
(batch, head-block) slices so that the L x L scores of only a few heads exist at a time, can
evaluate a subset of query rows, takes the optional additive mask of the operator
(src/fused_attn_extention.cu:21; added to the scaled scores of every head, README.md:88-89) and
can run in float64.

Pinned: tests/golden/*.npz hold outputs of the reference function itself (imported from the
reference tree by tests/golden/make_golden.py) and tests/test_oracle.py checks this file against
them.  The mask argument has no counterpart in the reference's naive function and no reference
test, so for masked calls parity is unpinned; they are checked against the formula above only.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch


def attention(queries: torch.Tensor, keys: torch.Tensor, values: torch.Tensor, head_dim: int,
              mask: Optional[torch.Tensor] = None, *, dtype: torch.dtype = torch.float32,
              query_rows: Optional[Sequence[int]] = None, max_score_elems: int = 1 << 27) -> torch.Tensor:
    """softmax(Q K^T / sqrt(head_dim)) V per head for [B, L, F] inputs; returns [B, Lq, F] in `dtype`.

    `query_rows` selects the query positions to evaluate (default: all L); keys and values are
    always used in full.
    """
    if queries.dim() != 3 or keys.shape != queries.shape or values.shape != queries.shape:
        raise ValueError("queries, keys, values must be [B, L, F] of one shape")
    B, L, F = queries.shape
    if F % head_dim:
        raise ValueError("F must be divisible by head_dim")
    R = F // head_dim
    rows = torch.arange(L) if query_rows is None else torch.as_tensor(list(query_rows), dtype=torch.long)
    Lq = rows.numel()
    q = queries.to(dtype).reshape(B, L, R, head_dim)
    k = keys.to(dtype).reshape(B, L, R, head_dim)
    v = values.to(dtype).reshape(B, L, R, head_dim)
    out = torch.empty(B, Lq, F, dtype=dtype)
    heads_per_block = max(1, min(R, max_score_elems // max(1, Lq * L)))
    root = head_dim ** 0.5
    for b in range(B):
        mrows = None if mask is None else mask[b].to(dtype)[rows]             # [Lq, L]
        for h0 in range(0, R, heads_per_block):
            h1 = min(R, h0 + heads_per_block)
            qh = q[b, :, h0:h1].index_select(0, rows).transpose(0, 1)          # [hb, Lq, H]
            kh = k[b, :, h0:h1].transpose(0, 1)                                # [hb, L, H]
            vh = v[b, :, h0:h1].transpose(0, 1)                                # [hb, L, H]
            scores = torch.matmul(qh, kh.transpose(1, 2)) / root               # [hb, Lq, L]
            if mrows is not None:
                scores = scores + mrows
            probs = torch.softmax(scores, dim=-1)
            o = torch.matmul(probs, vh)                                        # [hb, Lq, H]
            out[b, :, h0 * head_dim:h1 * head_dim] = o.transpose(0, 1).reshape(Lq, (h1 - h0) * head_dim)
    return out


def error_metrics(actual: torch.Tensor, expected: torch.Tensor) -> dict:
    """max-abs, mean-abs and rms-relative error of `actual` against `expected` (both upcast)."""
    a = actual.to(torch.float64)
    e = expected.to(torch.float64)
    d = (a - e).abs()
    rms = float(e.pow(2).mean().sqrt())
    return {"max_abs": float(d.max()), "mean_abs": float(d.mean()), "rms_ref": rms,
            "max_abs_over_rms": float(d.max()) / rms if rms > 0 else float("inf")}


# Tolerance of the operator against this oracle run in fp32 on the fp16-rounded inputs.
MAX_ABS_TOL = 2e-3
MEAN_ABS_TOL = 2e-4
