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


@pytest.mark.parametrize("B,R,L,H", [(4, 32, 2048, 128), (4, 16, 2048, 128), (4, 8, 2048, 128), (4, 4, 2048, 128),
                                     (8, 12, 512, 64), (64, 16, 197, 64), (1, 32, 16384, 128), (1, 4, 16384, 128),
                                     (2, 3, 818, 128), (1, 4, 2048, 128), (1, 2, 4096, 64), (5, 7, 700, 64),
                                     (1, 1, 100000, 128), (3, 50, 1000, 128), (2, 2, 700, 128)])
@pytest.mark.parametrize("sms", [148, 132, 16])
def test_every_key_step_of_every_work_item_is_scheduled_exactly_once(B, R, L, H, sms):
    """The kernel's schedule (whole items round-robin, a divided last round) restated in Python from
    what the launcher reports: full coverage, no overlap, and the limits the kernel relies on."""
    single = fa._lib.FLAG_FORCE_PIPELINED | fa._lib.FLAG_NO_PAIR      # the kernel on single CTAs
    sched = fa.describe_schedule(B, L, R * H, H, flags=single, sm_count=sms)
    n = sched["key_steps"]
    assert n == -(-L // 128)
    n_items = -(-L // 256) * R * B
    grid, T = sched["grid"], sched["tail_steps"]
    assert 1 <= grid <= sms
    seen = {}
    for cta in range(grid):
        segs = fa.cta_segments(sched, n_items, cta)
        tail = [s for s in segs if s[2] != n or s[0] >= sched["full_rounds"] * grid] if T else []
        assert len(tail) <= 2                                  # two scratch slots per CTA
        for item, j0, ln in segs:
            assert 0 <= item < n_items and ln >= 1 and j0 + ln <= n
            for j in range(j0, j0 + ln):
                assert (item, j) not in seen
                seen[(item, j)] = cta
    assert len(seen) == n_items * n
    if T:
        tg = sched["tail_grid"]
        assert T == sched["tail_items"] * n and 1 <= tg <= grid and T * tg < 2 ** 32
        assert sched["full_rounds"] * sms + sched["tail_items"] == n_items
        assert sched["full_rounds"] == 0 or grid == sms
        busiest = max(sum(s[2] for s in fa.cta_segments(sched, n_items, c)) for c in range(grid))
        whole_rounds = -(-n_items // sms) * n
        assert busiest < whole_rounds - 5 - max(1, whole_rounds // 20)    # only where it clearly pays (see the launcher)
        for item in range(sched["full_rounds"] * grid, n_items):
            ctas = sorted({seen[(item, j)] for j in range(n)})
            assert len(ctas) <= 3 and ctas == list(range(ctas[0], ctas[-1] + 1))   # consecutive CTAs, at most 3 parts
    # undivided on request
    whole = fa.describe_schedule(B, L, R * H, H, flags=single | fa._lib.FLAG_NO_SPLIT, sm_count=sms)
    assert whole["tail_steps"] == 0 and whole["grid"] == min(sms, n_items)


def test_headline_shards_are_divided_as_designed():
    d = lambda R: fa.describe_schedule(4, 2048, R * 128, 128, flags=fa._lib.FLAG_NO_PAIR)
    assert fa.describe_schedule(4, 2048, 32 * 128, 128) == {
        "kernel": "pipelined on pairs of CTAs", "grid": 148, "full_rounds": 7, "tail_items": 0, "tail_steps": 0,
        "key_steps": 16, "tail_grid": 0}                   # 512 work items of 512 rows on 74 pairs of SMs
    assert d(32)["tail_steps"] == 0                       # 6.92 rounds: the last one is nearly full
    # the shards of the headline job are not divided: what it would save (8, 4, 2 key steps at 2, 4, 8 GPUs) is
    # about what it costs
    assert d(16)["tail_steps"] == 0 and d(8)["tail_steps"] == 0 and d(4)["tail_steps"] == 0
    few = fa.describe_schedule(1, 2048, 4 * 128, 128)     # 32 items on 148 SMs: two CTAs per item
    assert (few["grid"], few["full_rounds"], few["tail_items"], few["tail_grid"]) == (64, 0, 32, 64)
    long = fa.describe_schedule(1, 16384, 4 * 128, 128)   # 256 items of 128 key steps: the last 108 are divided
    assert (long["full_rounds"], long["tail_items"], long["tail_grid"]) == (1, 108, 148)


def test_clock_count_records_are_parsed_and_summarised():
    """fused_attention_b200/cycles.py on a synthetic device buffer: records of launches in any slot order, empty
    slots skipped, medians of SM clocks, busy time, period and the gap between launches."""
    from fused_attention_b200 import cycles
    words = [0] * 256
    t0 = 1_000_000
    for n, slot in enumerate((5, 6, 7, 3)):        # launch ids wrap around the 64 records
        entry = t0 + n * 200_000
        words[4 * slot: 4 * slot + 4] = [entry, entry + 30_000, entry + 190_000, 300_000 + n]
    words[4 * 9: 4 * 9 + 4] = [77, 50, 60, 1]      # ready before entry: not a record
    recs = cycles.parse_records(words)
    assert [r["sm_clocks"] for r in recs] == [300_000, 300_001, 300_002, 300_003]
    s = cycles.summarise(recs)
    assert s["launches"] == 4 and s["sm_clocks"] == 300_002
    assert s["busy_us"] == 160.0 and s["period_us"] == 200.0 and s["gap_us"] == 40.0
    assert cycles.summarise([])["sm_clocks"] is None


def test_time_line_words_are_parsed():
    """cycles.parse_timeline on a synthetic buffer: key steps 2800 clocks apart, tile 1 lagging tile 0 by 1100,
    a softmax pass of 2560 clocks per tile; stamps of steps that were not reached stay zero and are skipped."""
    from fused_attention_b200 import cycles
    w = [0] * cycles.TIMELINE_WORDS

    def put(role, g, ev, v):
        w[256 + (role * 256 + g) * 8 + ev] = v
    for g in range(60):
        t = 10_000 + g * 2800
        for i in (0, 1):
            for ev, off in enumerate((0, 120, 150, 950, 1120, 2520, 2680)):
                put(i, g, ev, t + i * 1100 + off)
        for ev, off in enumerate((0, 200, 900, 1100, 2300, 2500)):
            put(2, g, ev, t + off - 600)
        for ev, off in enumerate((0, 200, 1200, 1400, 2300, 2500)):
            put(3, g, ev, t + off + 1500)
    r = cycles.parse_timeline(w, 20, 100)      # steps 60..99 were never reached
    assert r["steps_recorded"] == 60 and r["step_period"] == 2800.0
    assert r["tile0"]["pass"] == 2560.0 and r["tile1"]["wait_for_S"] == 120.0
    assert r["tile0"]["wait_for_P_buffer"] == 170.0 and r["tile0"]["hand_over"] == 160.0
    assert r["qk_warp"] == {"wait_for_K": 200.0, "wait_for_S_read_by_tile1": 700.0, "wait_for_S_read_by_tile0": 1200.0}
    assert r["pv_warp"]["wait_for_P0"] == 1000.0
    assert r["S_finished_before_its_tile_looks"]["tile0_issue_to_seen"] == 10_000 + 120 - (10_000 + 900 - 600)
    assert cycles.parse_timeline([0] * cycles.TIMELINE_WORDS)["step_period"] is None
