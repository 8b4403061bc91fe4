"""The CPU oracle against the reference's own outputs (golden vectors) and against first principles."""
import glob
import math
import os

import numpy as np
import pytest
import torch

from oracle.naive_attention import attention, error_metrics

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))


def test_golden_set_is_complete():
    names = {os.path.basename(p)[:-4] for p in GOLDEN}
    # the reference's twelve (head_dim, chunk_size) unit-test shapes, tests/test_fused_attn.py:33-67
    for H, C in ((16, 16), (16, 32), (32, 16), (32, 32), (32, 64), (64, 16), (64, 32), (64, 64), (64, 128),
                 (128, 32), (128, 64), (128, 128)):
        assert f"ref_test_h{H}_c{C}" in names
    assert {"tiny", "ragged_l197", "ragged_l300_h128", "short_l5_h32"} <= names


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_oracle_reproduces_reference_outputs(path):
    d = np.load(path)
    q, k, v = (torch.from_numpy(d[n]) for n in "qkv")
    y_ref = torch.from_numpy(d["y"])
    torch.set_num_threads(1)
    y = attention(q, k, v, int(d["head_dim"]))
    assert y.shape == y_ref.shape and y.dtype == torch.float32
    # same torch primitives in the same order: differences are at most a few ulps of fp32
    assert float((y - y_ref).abs().max()) <= 2e-6


def _attention_by_hand(q, k, v, H, mask=None):
    """Scalar-loop definition, float64: for checking the oracle on tiny inputs."""
    B, L, F = q.shape
    out = np.zeros((B, L, F))
    qd, kd, vd = (t.double().numpy() for t in (q, k, v))
    for b in range(B):
        for h in range(F // H):
            c = slice(h * H, (h + 1) * H)
            for i in range(L):
                s = np.array([qd[b, i, c] @ kd[b, j, c] / math.sqrt(H) for j in range(L)])
                if mask is not None:
                    s = s + mask[b, i].double().numpy()
                w = np.exp(s - s.max())
                w /= w.sum()
                out[b, i, c] = w @ vd[b, :, c]
    return torch.from_numpy(out)


def test_oracle_matches_scalar_definition():
    g = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn(2, 7, 48, generator=g).half() for _ in range(3))
    y = attention(q, k, v, 16, dtype=torch.float64)
    assert float((y - _attention_by_hand(q, k, v, 16)).abs().max()) < 1e-12


def test_oracle_mask_matches_scalar_definition():
    g = torch.Generator().manual_seed(6)
    q, k, v = (torch.randn(2, 9, 32, generator=g).half() for _ in range(3))
    mask = torch.zeros(2, 9, 9, dtype=torch.float16)
    mask[:, :, 5:] = float("-inf")          # padding mask
    mask[0] += torch.triu(torch.full((9, 9), float("-inf")), diagonal=1).half()  # causal for batch 0
    y = attention(q, k, v, 16, mask, dtype=torch.float64)
    assert float((y - _attention_by_hand(q, k, v, 16, mask)).abs().max()) < 1e-12


def test_query_rows_subset_and_blocking():
    g = torch.Generator().manual_seed(7)
    q, k, v = (torch.randn(2, 50, 64, generator=g).half() for _ in range(3))
    full = attention(q, k, v, 16)
    rows = [0, 3, 49, 17]
    sub = attention(q, k, v, 16, query_rows=rows)
    assert torch.equal(sub, full[:, rows])
    # one head at a time gives the same numbers as all heads at once
    one = attention(q, k, v, 16, max_score_elems=1)
    assert float((one - full).abs().max()) <= 1e-6


def test_fp32_oracle_close_to_fp64():
    g = torch.Generator().manual_seed(8)
    q, k, v = (torch.randn(1, 300, 128, generator=g).half() for _ in range(3))
    m = error_metrics(attention(q, k, v, 64), attention(q, k, v, 64, dtype=torch.float64))
    assert m["max_abs"] < 1e-5
