"""Host-side logic that needs no GPU: argument checks of the operator mirror, sharding, workloads."""
import itertools
import os
import sys

import pytest
import torch

import fused_attention_b200 as fa
from fused_attention_b200.workloads import WORKLOADS, make_inputs, workload_inputs


def _t(*shape, dtype=torch.float16):
    return torch.zeros(*shape, dtype=dtype)


def test_cpu_tensors_are_rejected_like_the_reference_binding():
    # src/fused_attn_extention.cu:24-43 -> RuntimeError; there is no CPU path to fall back to
    with pytest.raises(RuntimeError, match="CUDA"):
        fa.attention_forward(64, 64, _t(1, 64, 64), _t(1, 64, 64), _t(1, 64, 64))
    with pytest.raises(RuntimeError, match="float16"):
        fa.attention_forward(64, 64, _t(1, 64, 64, dtype=torch.float32), _t(1, 64, 64), _t(1, 64, 64))
    with pytest.raises(RuntimeError):
        fa.attention_forward(64, 64, _t(64, 64), _t(1, 64, 64), _t(1, 64, 64))


def test_torch_extension_module_surface():
    ext_dir = os.path.join(os.path.dirname(fa.__file__), "ext")
    if not any(f.startswith("fused_attn") and f.endswith(".so") for f in os.listdir(ext_dir) if os.path.isdir(ext_dir)):
        pytest.skip("extension module not built")
    sys.path.insert(0, ext_dir)
    import fused_attn  # noqa: E402  (torch is imported first, as the reference README requires)
    doc = fused_attn.attention_forward.__doc__
    for name in ("head_dim", "chunk_size", "queries", "keys", "values", "mask"):
        assert name in doc
    with pytest.raises(RuntimeError):
        fused_attn.attention_forward(64, 64, _t(1, 64, 64), _t(1, 64, 64), _t(1, 64, 64))
    with pytest.raises(RuntimeError):
        fused_attn.attention_forward(head_dim=64, chunk_size=64, queries=_t(1, 64, 64), keys=_t(1, 64, 64),
                                     values=_t(1, 64, 64), mask=None)


@pytest.mark.parametrize("B,R", [(4, 32), (1, 32), (8, 12), (64, 16), (1, 4), (3, 5), (2, 7)])
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_shards_cover_every_unit_exactly_once(B, R, world):
    seen = set()
    for rank in range(world):
        s = fa.shard_units(B, R, world, rank)
        for u in itertools.product(range(s.b0, s.b1), range(s.h0, s.h1)):
            assert u not in seen
            seen.add(u)
    assert seen == set(itertools.product(range(B), range(R)))


def test_shard_rules():
    assert fa.shard_units(4, 32, 8, 3) == fa.Shard(0, 4, 12, 16)          # heads when R % n == 0
    assert fa.shard_units(8, 12, 8, 5) == fa.Shard(5, 6, 0, 12)           # else batches
    assert [fa.shard_units(1, 5, 4, r).units for r in range(4)] == [2, 1, 1, 1]
    with pytest.raises(ValueError):
        fa.shard_units(1, 4, 2, 2)


def test_slice_tensor_matches_head_columns():
    t = torch.arange(2 * 3 * 8 * 4).reshape(2, 3, 32).half()
    s = fa.Shard(0, 2, 2, 5)
    got = fa.slice_tensor(t, s, 4)
    assert got.is_contiguous() and got.shape == (2, 3, 12)
    assert torch.equal(got, t[:, :, 8:20])


def test_workload_accounting_matches_the_specification():
    w = WORKLOADS
    assert w["tiny"].flops == pytest.approx(6.711e7, rel=1e-3)
    assert w["bert_base"].flops == pytest.approx(6.442e9, rel=1e-3)
    assert w["vit_l16_ragged"].flops == pytest.approx(1.0174e10, rel=1e-3)
    assert w["llama7b_prefill"].flops == pytest.approx(2.7488e11, rel=1e-3)
    assert w["long_context"].flops == pytest.approx(4.3980e12, rel=1e-3)
    assert w["llama7b_prefill"].bytes == pytest.approx(268.4e6, rel=1e-3)
    assert fa.attention_flops(4, 32, 2048, 128) == w["llama7b_prefill"].flops
    assert fa.attention_bytes(4, 32, 2048, 128) == w["llama7b_prefill"].bytes


def test_inputs_are_seeded_and_sliced_consistently():
    a = make_inputs(2, 10, 64, 0.5, 7)
    b = make_inputs(2, 10, 64, 0.5, 7)
    assert all(torch.equal(x, y) for x, y in zip(a, b))
    assert a[0].dtype == torch.float16 and abs(float(a[0].float().std()) - 0.5) < 0.05
    w = WORKLOADS["tiny"]
    full = workload_inputs(w)
    part = workload_inputs(w, heads=slice(1, 3))
    assert torch.equal(part[1], full[1][:, :, 64:192])
