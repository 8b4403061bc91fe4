"""Parity of the CUDA path (through the C ABI) with the CPU oracle and the reference's golden outputs.

Tolerance (fp16 operator against the fp32 oracle on the same fp16-rounded inputs):
max-abs <= 2e-3 and mean-abs <= 2e-4.
"""
import ctypes
import glob
import os
import sys

import numpy as np
import pytest
import torch

import fused_attention_b200 as fa
from fused_attention_b200 import _lib
from fused_attention_b200.workloads import WORKLOADS, make_inputs, workload_inputs
from oracle.naive_attention import MAX_ABS_TOL, MEAN_ABS_TOL, attention as oracle, error_metrics

pytestmark = pytest.mark.gpu

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))
SIMPLE, PIPE, WHOLE = _lib.FLAG_FORCE_SIMPLE, _lib.FLAG_FORCE_PIPELINED, _lib.FLAG_NO_SPLIT
PAIR = _lib.FLAG_FORCE_PAIR                      # head_dim 128 on pairs of CTAs (one MMA of 256 rows for two SMs)
ONE = PIPE | _lib.FLAG_NO_PAIR                   # the warp-specialised kernel on single CTAs


def run(q, k, v, H, mask=None, flags=0, chunk=None):
    chunk = chunk or (32 if H == 128 else 16)
    out = fa.attention_forward(H, chunk, q.cuda(), k.cuda(), v.cuda(),
                               None if mask is None else mask.cuda(), flags=flags | _lib.FLAG_SYNC)
    return out.float().cpu()


def assert_close(y, expected):
    assert not torch.isnan(y).any()
    m = error_metrics(y, expected)
    assert m["max_abs"] <= MAX_ABS_TOL, m
    assert m["mean_abs"] <= MEAN_ABS_TOL, m
    return m


@pytest.fixture(autouse=True)
def status_word_stays_clear():
    yield
    assert fa.read_status(0) == (0, 0)


def kernels_for(H, L=1024):
    return [0, SIMPLE] + ([ONE] if H >= 64 else []) + ([PAIR] if H == 128 else [])


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_golden_vectors_of_the_reference(path):
    d = np.load(path)
    q, k, v = (torch.from_numpy(d[n]) for n in "qkv")
    H = int(d["head_dim"])
    for flags in kernels_for(H):
        assert_close(run(q, k, v, H, flags=flags), torch.from_numpy(d["y"]))


@pytest.mark.parametrize("name", ["tiny", "bert_base", "vit_l16_ragged"])
def test_benchmark_configurations_full_oracle(name):
    w = WORKLOADS[name]
    q, k, v = workload_inputs(w)
    expected = oracle(q, k, v, w.H)
    for flags in kernels_for(w.H):
        assert_close(run(q, k, v, w.H, flags=flags), expected)


@pytest.mark.parametrize("name", ["llama7b_prefill", "long_context"])
def test_full_size_configurations_sampled_rows(name):
    """Every head and batch, 96 seeded query rows (plus first and last) against all keys."""
    w = WORKLOADS[name]
    q, k, v = workload_inputs(w)
    g = torch.Generator().manual_seed(w.seed)
    rows = sorted(set(torch.randint(0, w.L, (96,), generator=g).tolist()) | {0, 127, 128, w.L - 1})
    expected = oracle(q, k, v, w.H, query_rows=rows)
    rms = float(expected.double().pow(2).mean().sqrt())
    for flags in (0, SIMPLE):
        y = run(q, k, v, w.H, flags=flags)[:, rows]
        m = assert_close(y, expected)
        # outputs are small at these shapes: also bound the error relative to rms(Y)
        assert m["max_abs"] / rms < 2e-2, m


def _fp32_attention_on_device(q, k, v, H, b, h):
    """softmax(q k^T / sqrt(H)) v of one (batch, head) in fp32 on the GPU, in blocks of 2048 query rows."""
    qf, kf, vf = (t[b, :, h * H:(h + 1) * H].float() for t in (q, k, v))
    out = torch.empty_like(qf)
    for r0 in range(0, qf.shape[0], 2048):
        out[r0:r0 + 2048] = torch.softmax(qf[r0:r0 + 2048] @ kf.T / H ** 0.5, -1) @ vf
    return out


@pytest.mark.parametrize("name", ["llama7b_prefill", "long_context"])
def test_full_size_configurations_every_row(name):
    """Every query row of every (batch, head) of the two large configurations, all three kernels, against
    fp32 attention computed on the same GPU (the CPU oracle would need minutes to hours at these sizes);
    that checker is itself held against the CPU oracle on sampled rows of every head."""
    w = WORKLOADS[name]
    hq, hk, hv = workload_inputs(w)
    q, k, v = hq.cuda(), hk.cuda(), hv.cuda()
    g = torch.Generator().manual_seed(w.seed + 1)
    rows = sorted(set(torch.randint(0, w.L, (24,), generator=g).tolist()) | {0, w.L - 1})
    cpu = oracle(hq, hk, hv, w.H, query_rows=rows)                 # [B, rows, F]
    kernels = (ONE, PAIR, SIMPLE)
    ys = {flags: fa.attention_forward(w.H, 128, q, k, v, flags=flags) for flags in kernels}
    torch.cuda.synchronize()
    worst = {flags: [0.0, 0.0] for flags in kernels}
    checker_worst = 0.0
    for b in range(w.B):
        for h in range(w.R):
            ref = _fp32_attention_on_device(q, k, v, w.H, b, h)
            checker_worst = max(checker_worst, float((ref[rows].cpu() - cpu[b, :, h * w.H:(h + 1) * w.H]).abs().max()))
            for flags, y in ys.items():
                d = (y[b, :, h * w.H:(h + 1) * w.H].float() - ref).abs()
                worst[flags][0] = max(worst[flags][0], float(d.max()))
                worst[flags][1] = max(worst[flags][1], float(d.mean()))
    assert checker_worst <= 2e-5, checker_worst      # fp32 against fp32: only the order of summation differs
    for flags in kernels:
        assert worst[flags][0] <= MAX_ABS_TOL and worst[flags][1] <= MEAN_ABS_TOL, (flags, worst[flags])


@pytest.mark.parametrize("H", [16, 32, 64, 128])
@pytest.mark.parametrize("L", [1, 2, 31, 127, 128, 129, 255, 256, 257, 383, 385, 640])
def test_ragged_lengths(H, L):
    q, k, v = make_inputs(2, L, 3 * H, 1.0, 1000 + L)
    expected = oracle(q, k, v, H)
    for flags in kernels_for(H):
        assert_close(run(q, k, v, H, flags=flags), expected)


def _fuzz_cases():
    import random
    rng = random.Random(20261125)
    cases = []
    for _ in range(24):
        H = rng.choice([16, 32, 64, 64, 128, 128])
        B = rng.randint(1, 5)
        R = rng.randint(1, 9)
        L = rng.choice([rng.randint(1, 130), rng.randint(131, 700), rng.randint(701, 1500)])
        flags = rng.choice([0, SIMPLE] + ([PIPE, PIPE] if H >= 64 else []))
        sigma = rng.choice([0.5, 1.0, 2.0])
        cases.append((H, B, R, L, flags, sigma))
    return cases


@pytest.mark.parametrize("H,B,R,L,flags,sigma", _fuzz_cases())
def test_seeded_random_shapes(H, B, R, L, flags, sigma):
    q, k, v = make_inputs(B, L, R * H, sigma, 7000 + L + H)
    expected = oracle(q, k, v, H)
    y = run(q, k, v, H, flags=flags)
    m = error_metrics(y, expected)
    scale = max(1.0, sigma)          # |V| grows with sigma; the bound is for unit-scale values
    assert m["max_abs"] <= MAX_ABS_TOL * scale and m["mean_abs"] <= MEAN_ABS_TOL * scale, m


@pytest.mark.parametrize("seed", [1, 2])
def test_many_random_shapes_against_fp32_attention_on_the_device(seed):
    """200 shapes per seed (lengths to 5000, up to 40 heads, key spikes that move the reference maximum
    late in a tile) through the pipelined kernel; the checker here is fp32 torch attention on the same GPU
    because the CPU oracle would need minutes at these sizes. Tolerance: the absolute bound for unit-scale
    values, times sigma, plus one fp16 rounding of the output value itself; results must repeat bit for bit."""
    import random
    rng = random.Random(seed)
    failures = []
    for it in range(200):
        H = rng.choice([64, 128])
        B = rng.randint(1, 6)
        R = rng.randint(1, 40)
        L = rng.choice([rng.randint(1, 300), rng.randint(300, 1500), rng.randint(1500, 5000)])
        if B * R * L * L > 3e9:
            R = max(1, int(3e9 / (B * L * L)))
        sigma = rng.choice([0.3, 1.0, 2.5])
        g = torch.Generator(device="cuda")
        g.manual_seed(1000 * seed + it)
        q, k, v = ((torch.randn(B, L, R * H, generator=g, device="cuda") * sigma).half() for _ in range(3))
        if rng.random() < 0.3:
            pos = rng.randrange(L)
            k[:, pos, :] = 3.0 * q[:, rng.randrange(L), :].sign()
        y = fa.attention_forward(H, 32, q, k, v, flags=PIPE)
        y2 = fa.attention_forward(H, 32, q, k, v, flags=PIPE)
        qf, kf, vf = (t.float().view(B, L, R, H).transpose(1, 2) for t in (q, k, v))
        ref = (torch.softmax(qf @ kf.mT / H ** 0.5, -1) @ vf).transpose(1, 2).reshape(B, L, R * H)
        d = (y.float() - ref).abs()
        excess = (d - (MAX_ABS_TOL * max(1.0, sigma) + ref.abs() * 2.0 ** -10)).max().item()
        if not (torch.isfinite(y).all().item() and excess <= 0 and torch.equal(y, y2)):
            failures.append((H, B, R, L, sigma, d.max().item()))
    assert not failures, failures


def test_many_random_shapes_with_a_mask_against_fp32_attention_on_the_device():
    """80 shapes with an additive mask (causal, or a padded tail, plus soft values) at head_dim 64 and 128 through
    whatever kernel the launcher picks: lengths that are multiples of 8 (mask tiles through TMA, on pairs of CTAs
    or on single ones) and lengths that are not (rows read from global memory); checker and tolerance as above."""
    import random
    rng = random.Random(7)
    failures = []
    for it in range(80):
        H = rng.choice([64, 128])
        B = rng.randint(1, 4)
        R = rng.randint(1, 24)
        L = rng.choice([rng.randint(1, 300), rng.randint(300, 1500), rng.randint(1500, 3000)])
        if rng.random() < 0.6:
            L = max(8, L // 8 * 8)
        if B * R * L * L > 1.5e9:
            R = max(1, int(1.5e9 / (B * L * L)))
        g = torch.Generator(device="cuda")
        g.manual_seed(5000 + it)
        q, k, v = (torch.randn(B, L, R * H, generator=g, device="cuda").half() for _ in range(3))
        mask = (0.5 * torch.randn(B, L, L, generator=g, device="cuda")).half()
        if rng.random() < 0.5:
            mask += torch.triu(torch.full((L, L), float("-inf"), device="cuda", dtype=torch.float16), diagonal=1)
        else:
            mask[:, :, L - L // 3:] = float("-inf") if L >= 3 else 0.0
        y = fa.attention_forward(H, 32, q, k, v, mask)
        y2 = fa.attention_forward(H, 32, q, k, v, mask)
        qf, kf, vf = (t.float().view(B, L, R, H).transpose(1, 2) for t in (q, k, v))
        ref = (torch.softmax(qf @ kf.mT / H ** 0.5 + mask.float()[:, None], -1) @ vf).transpose(1, 2).reshape(B, L, R * H)
        d = (y.float() - ref).abs()
        excess = (d - (MAX_ABS_TOL + ref.abs() * 2.0 ** -10)).max().item()
        if not (torch.isfinite(y).all().item() and excess <= 0 and torch.equal(y, y2)):
            failures.append((H, B, R, L, d.max().item(), fa.select_kernel(B, L, R * H, H, has_mask=True)))
    assert not failures, failures


def test_many_batches_and_heads_index_correctly():
    # every (batch, head) pair gets its own inputs; a wrong offset shows as a large error
    q, k, v = make_inputs(5, 200, 7 * 64, 1.0, 77)
    expected = oracle(q, k, v, 64)
    for flags in (SIMPLE, PIPE):
        assert_close(run(q, k, v, 64, flags=flags), expected)


@pytest.mark.parametrize("flags", [PIPE, SIMPLE])
def test_tensors_larger_than_four_gib(flags):
    """Q, K, V and Y of 4.25 GiB each: the last batch entries lie beyond a 32-bit byte offset and the very
    last one beyond a 32-bit element offset (the reference indexes with 32-bit offsets,
    include/fused_attn.cuh:685-686, and cannot take this shape).  A batch entry of the big call must equal,
    bit for bit, the same entry computed alone, and that one is checked against fp32 attention."""
    B, L, F = 17, 4096, 32768                  # 17 * 4096 * 32768 = 2^31 + 2^27 elements
    H = 128 if flags == PIPE else 64
    R = F // H
    g = torch.Generator(device="cuda")
    g.manual_seed(4242)
    q, k, v = (torch.empty(B, L, F, dtype=torch.float16, device="cuda") for _ in range(3))
    for t in (q, k, v):
        for b in range(B):                     # filled entry by entry: no fp32 temporary of the whole tensor
            t[b] = torch.randn(L, F, generator=g, device="cuda", dtype=torch.float16)
    y = fa.attention_forward(H, 32 if H == 128 else 16, q, k, v, flags=flags | WHOLE)
    for b in (0, 8, B - 1):
        alone = fa.attention_forward(H, 32 if H == 128 else 16, q[b:b + 1], k[b:b + 1], v[b:b + 1], flags=flags | WHOLE)
        assert torch.equal(y[b], alone[0]), b
    # the default schedule may divide the key axis of the last work items of a call among CTAs: same values up
    # to the kernel's ordinary rounding error
    y_div = fa.attention_forward(H, 32 if H == 128 else 16, q, k, v, flags=flags)
    assert float((y_div[B - 1].float() - y[B - 1].float()).abs().max()) <= MAX_ABS_TOL / 4
    y = y_div
    b = B - 1
    for h in (0, R // 2, R - 1):               # heads at both ends of the last entry against fp32 attention
        qf, kf, vf = (t[b, :, h * H:(h + 1) * H].float() for t in (q, k, v))
        ref = torch.softmax(qf @ kf.T / H ** 0.5, -1) @ vf
        d = (y[b, :, h * H:(h + 1) * H].float() - ref).abs()
        assert d.max().item() <= MAX_ABS_TOL and d.mean().item() <= MEAN_ABS_TOL, (h, d.max().item())
    del q, k, v, y
    torch.cuda.empty_cache()


@pytest.mark.parametrize("B,R,L,H", [(40, 8, 100, 64), (40, 8, 200, 64), (20, 10, 300, 128), (3, 100, 130, 64),
                                     (2, 160, 257, 128)])
def test_persistent_kernel_with_several_items_per_cta(B, R, L, H):
    """More work items than SMs with one, two or three key steps each: every CTA of the persistent
    kernel walks several items, so the hand-overs between items (query buffers, O tiles, row sums)
    are exercised at their tightest."""
    q, k, v = make_inputs(B, L, R * H, 1.0, 2000 + L)
    expected = oracle(q, k, v, H)
    assert_close(run(q, k, v, H, flags=PIPE), expected)


def _device_fp32(q, k, v, H):
    B, L, F = q.shape
    qf, kf, vf = (t.float().view(B, L, F // H, H).transpose(1, 2) for t in (q, k, v))
    return (torch.softmax(qf @ kf.mT / H ** 0.5, -1) @ vf).transpose(1, 2).reshape(B, L, F)


@pytest.mark.parametrize("B,R,L,H", [(1, 4, 2048, 128), (1, 2, 5000, 64), (1, 1, 4096, 128), (1, 3, 16384 + 77, 128),
                                     (1, 40, 3000, 64), (2, 5, 2000, 64), (1, 4, 16384, 128), (1, 16, 8192, 128),
                                     (1, 8, 8192, 64), (1, 3, 2300, 64), (1, 6, 3000, 128), (1, 7, 2500, 128)])
def test_last_round_divided_among_ctas(B, R, L, H):
    """Shapes whose work items do not fill a whole number of rounds of the persistent kernel: the key axis
    of the last round's items is divided among CTAs and the parts are merged in fp32.  Against fp32
    attention on the same GPU, against the same call with whole items, and twice for the bits."""
    sched = fa.describe_schedule(B, L, R * H, H, sm_count=fa.query(0)["sm_count"])
    assert sched["kernel"] == "pipelined" and sched["tail_steps"] > 0, sched
    g = torch.Generator(device="cuda")
    g.manual_seed(L + R)
    q, k, v = (torch.randn(B, L, R * H, generator=g, device="cuda").half() for _ in range(3))
    y = fa.attention_forward(H, 32, q, k, v, flags=_lib.FLAG_SYNC)
    y2 = fa.attention_forward(H, 32, q, k, v, flags=_lib.FLAG_SYNC)
    y_whole = fa.attention_forward(H, 32, q, k, v, flags=WHOLE | _lib.FLAG_SYNC)
    assert torch.equal(y, y2)                                   # the merge order is fixed: no run-to-run noise
    ref = _device_fp32(q, k, v, H)
    d = (y.float() - ref).abs()
    assert torch.isfinite(y).all()
    assert float(d.max()) <= MAX_ABS_TOL and float(d.mean()) <= MEAN_ABS_TOL, (float(d.max()), float(d.mean()))
    # Against the undivided schedule: every part takes its exponentials against its own reference maximum, so
    # the fp16 roundings of P differ between the two schedules; the results differ by the kernel's ordinary
    # rounding error (observed up to 1e-4), a fraction of the bound against the oracle.
    assert float((y.float() - y_whole.float()).abs().max()) <= MAX_ABS_TOL / 4


@pytest.mark.parametrize("H", [64, 128])
@pytest.mark.parametrize("pattern", ["rising", "falling", "spike"])
def test_divided_items_whose_parts_have_far_apart_maxima(H, pattern):
    """The parts of a divided item each keep their own reference maximum; here the maxima of the parts lie
    hundreds of powers of two apart (rising or falling score levels along the keys, or one late spike), so
    the weights of the merge range from 1 down to 0."""
    B, R, L = 1, 4, 128 * 16 + 50
    assert fa.describe_schedule(B, L, R * H, H, sm_count=fa.query(0)["sm_count"])["tail_steps"] > 0
    q, k, v = make_inputs(B, L, R * H, 1.0, 4100 + H)
    q = (q.float() * 0.05 + 1.0).half()
    tile = torch.arange(L) // 128
    if pattern == "rising":
        level = 40.0 * tile
    elif pattern == "falling":
        level = 40.0 * (tile.max() - tile)
    else:
        level = torch.zeros(L); level[128 * 11 + 77] = 400.0
    k = (k.float() * 0.05 + (level / H)[None, :, None]).half()
    expected = oracle(q, k, v, H)
    y = run(q, k, v, H)
    assert torch.isfinite(y).all()
    assert_close(y, expected)
    assert_close(run(q, k, v, H, flags=WHOLE), expected)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_a_shard_reproduces_the_bits_of_the_undivided_job(world):
    """Strong scaling by head: with FA_B200_FLAG_NO_SPLIT the heads of a shard have the bits they have in the
    one-GPU job (each (batch, head) is computed the same way whatever else is in the call); the default
    schedule, which may divide the key axis of some work items, stays within the kernel's rounding error of it."""
    w = WORKLOADS["llama7b_prefill"]
    q, k, v = (t.cuda() for t in workload_inputs(w))
    y_full = fa.attention_forward(w.H, 128, q, k, v, flags=WHOLE)
    for rank in (0, world - 1):
        sh = fa.shard_units(w.B, w.R, world, rank)
        sq, sk, sv = (fa.slice_tensor(t, sh, w.H) for t in (q, k, v))
        want = y_full[sh.b0:sh.b1, :, sh.h0 * w.H:sh.h1 * w.H]
        assert torch.equal(fa.attention_forward(w.H, 128, sq, sk, sv, flags=WHOLE), want)
        got = fa.attention_forward(w.H, 128, sq, sk, sv).float()
        assert float((got - want.float()).abs().max()) <= MAX_ABS_TOL / 4


@pytest.mark.parametrize("B,R,L", [(1, 1, 1), (1, 1, 128), (1, 2, 129), (2, 3, 511), (2, 3, 512), (2, 3, 513), (1, 2, 1000),
                                   (20, 10, 300), (3, 50, 700), (4, 32, 2048), (1, 3, 5000), (1, 1, 16384 + 77)])
def test_kernel_on_pairs_of_ctas(B, R, L):
    """head_dim 128 on clusters of two CTAs: a pair works on 512 query rows and every MMA is one instruction
    of 256 rows for both SMs.  Lengths around the 512-row and 128-key boundaries, more work items than
    pairs of SMs, a single item.  Same arithmetic in the same order as the single-CTA kernel: same bits."""
    H = 128
    g = torch.Generator(device="cuda")
    g.manual_seed(L + R)
    q, k, v = (torch.randn(B, L, R * H, generator=g, device="cuda").half() for _ in range(3))
    y = fa.attention_forward(H, 128, q, k, v, flags=PAIR | _lib.FLAG_SYNC)
    assert torch.isfinite(y).all()
    d = (y.float() - _device_fp32(q, k, v, H)).abs()
    assert float(d.max()) <= MAX_ABS_TOL and float(d.mean()) <= MEAN_ABS_TOL, (float(d.max()), float(d.mean()))
    assert torch.equal(y, fa.attention_forward(H, 128, q, k, v, flags=ONE | WHOLE | _lib.FLAG_SYNC))


def test_large_logits_stay_finite():
    # sigma 4 at H=128 gives scores of a few hundred before scaling: exercises the running max
    q, k, v = make_inputs(1, 512, 256, 4.0, 5)
    expected = oracle(q, k, v, 128)
    for flags in (SIMPLE, ONE, PAIR):
        y = run(q, k, v, 128, flags=flags)
        assert torch.isfinite(y).all()
        m = error_metrics(y, expected)
        assert m["max_abs"] <= 2e-2 and m["mean_abs"] <= 2e-3, m   # |V| reaches 16 here


@pytest.mark.parametrize("H", [64, 128])
@pytest.mark.parametrize("pattern", ["rising", "falling", "spike", "spike_in_last_keys_of_a_tile", "rising_by_32_keys"])
def test_reference_maximum_moves_between_key_tiles(H, pattern):
    """Scores that jump by far more than 2^8 (in the exp2 domain) from one key tile to the next:
    rising (every tile forces a new reference and an O rescale), falling (the first reference stays,
    later P underflow to zero) and a single late spike.  The pipelined kernel takes the exponentials of
    a key tile against the reference it already has, in chunks of 32 keys, and only redoes them when a
    score exceeds that reference by more than 2^8; the last two patterns put the new maximum into the
    last chunk of a tile, or make it move with every chunk."""
    B, R, L = 2, 3, 128 * 6 + 50
    q, k, v = make_inputs(B, L, R * H, 1.0, 4000 + H)
    q = (q.float() * 0.05 + 1.0).half()                      # close to all-ones queries
    tile = torch.arange(L) // 128
    if pattern == "rising":
        level = 70.0 * tile
    elif pattern == "falling":
        level = 70.0 * (tile.max() - tile)
    elif pattern == "spike":
        level = torch.zeros(L); level[128 * 4 + 17] = 300.0
    elif pattern == "spike_in_last_keys_of_a_tile":
        level = torch.zeros(L); level[128 * 3 + 101] = 300.0; level[128 * 5 + 127] = 450.0
    else:
        level = 70.0 * (torch.arange(L) // 32)
    k = (k.float() * 0.05 + (level / H)[None, :, None]).half()   # raw score of key j is about level[j]
    expected = oracle(q, k, v, H)
    for flags in (SIMPLE, ONE) + ((PAIR,) if H == 128 else ()):
        y = run(q, k, v, H, flags=flags)
        assert torch.isfinite(y).all()
        assert_close(y, expected)


def test_kernels_agree_and_are_deterministic():
    q, k, v = make_inputs(2, 700, 256, 1.0, 11)
    a = run(q, k, v, 128, flags=PIPE)
    b = run(q, k, v, 128, flags=PIPE)
    c = run(q, k, v, 128, flags=SIMPLE)
    assert torch.equal(a, b)
    assert float((a - c).abs().max()) <= 1e-3


@pytest.mark.parametrize("H,L,flags", [(128, 700, ONE), (128, 700, PAIR), (64, 300, PIPE), (64, 100, SIMPLE), (32, 200, SIMPLE)])
def test_overlapped_launches_keep_the_order_of_the_stream(H, L, flags):
    """By default a launch may become resident while the previous kernel of the stream drains.  A chain of
    launches in which each one reads what the one before wrote (Y of step i is V of step i + 1, with no
    synchronisation in between) must give the bits of the same chain run with plain launches, and a kernel
    of another library between two launches must be ordered as well."""
    q, k, v = (t.cuda() for t in make_inputs(3, L, 4 * H, 1.0, 31))
    chunk = 32 if H == 128 else 16

    def chain(extra):
        cur = v
        for step in range(12):
            cur = fa.attention_forward(H, chunk, q, k, cur, flags=flags | extra)
            if step % 4 == 3:
                cur = cur * 2            # a foreign kernel in the middle of the chain
        torch.cuda.synchronize()
        return cur

    overlapped = chain(0)
    plain = chain(_lib.FLAG_NO_OVERLAP)
    assert torch.equal(overlapped, plain)
    assert torch.isfinite(overlapped).all()


@pytest.mark.parametrize("H", [16, 64, 128])
@pytest.mark.parametrize("L", [64, 200, 300])
def test_additive_mask(H, L):
    """Mask applied to every key tile; parity with the reference is unpinned for masks (its naive
    function takes none), so the oracle's formula scores + mask is the definition."""
    q, k, v = make_inputs(2, L, 2 * H, 1.0, 300 + L)
    mask = torch.zeros(2, L, L, dtype=torch.float16)
    mask[0] = torch.triu(torch.full((L, L), float("-inf")), diagonal=1).half()   # causal
    mask[1, :, L - L // 3:] = float("-inf")                                        # padding
    mask[1, :, : L // 2] += 0.5 * torch.randn(L, L // 2, generator=torch.Generator().manual_seed(1)).half()
    expected = oracle(q, k, v, H, mask)
    # the kernel on pairs of CTAs takes a mask only through TMA: rows of 16-byte multiples
    for flags in [f for f in kernels_for(H) if f != PAIR or L % 8 == 0]:
        assert_close(run(q, k, v, H, mask=mask, flags=flags), expected)


@pytest.mark.parametrize("L", [127, 200, 256, 1000])
def test_additive_mask_rows_at_any_alignment(L):
    """Mask rows are read with 16-byte loads when they start on a 16-byte boundary and value by value
    otherwise (L not a multiple of 8, or a mask tensor that starts at an odd element)."""
    H = 64
    q, k, v = make_inputs(2, L, 3 * H, 1.0, 600 + L)
    gen = torch.Generator().manual_seed(L)
    mask = (0.5 * torch.randn(2, L, L, generator=gen)).half()
    mask[0] += torch.triu(torch.full((L, L), float("-inf")), diagonal=1).half()
    expected = oracle(q, k, v, H, mask)
    for flags in (SIMPLE, PIPE):
        assert_close(run(q, k, v, H, mask=mask, flags=flags), expected)
    # the same values in a buffer whose first element is 2 bytes past a 16-byte boundary
    store = torch.empty(mask.numel() + 8, dtype=torch.float16, device="cuda")
    shifted = store[1:1 + mask.numel()].view_as(mask)
    shifted.copy_(mask)
    assert shifted.data_ptr() % 16 == 2
    for flags in (SIMPLE, PIPE):
        y = fa.attention_forward(H, 16, q.cuda(), k.cuda(), v.cuda(), shifted, flags=flags | _lib.FLAG_SYNC)
        assert_close(y.float().cpu(), expected)


@pytest.mark.parametrize("B,R,L,H", [(2, 8, 2048, 128), (2, 8, 2048, 64), (4, 32, 2048, 128), (1, 3, 1000, 128), (3, 4, 1336, 64)])
def test_additive_mask_on_long_sequences(B, R, L, H):
    """The warp-specialised kernels bring the mask in tile by tile through TMA (on single CTAs into one buffer that
    the two query tiles use in turn, on pairs of CTAs into a buffer per query tile); many key steps and many work
    items per CTA, where the two tiles drift apart in time.  Causal mask plus a soft random part; against fp32
    attention with the mask on the same GPU, and the two kernels against each other bit for bit."""
    g = torch.Generator(device="cuda")
    g.manual_seed(L + H)
    q, k, v = (torch.randn(B, L, R * H, generator=g, device="cuda").half() * 0.5 for _ in range(3))
    mask = torch.triu(torch.full((L, L), float("-inf"), device="cuda", dtype=torch.float16), diagonal=1)
    mask = mask.unsqueeze(0).repeat(B, 1, 1)
    mask += (0.5 * torch.randn(B, L, L, generator=g, device="cuda")).half()
    y = fa.attention_forward(H, 32, q, k, v, mask, flags=ONE | _lib.FLAG_SYNC)
    y2 = fa.attention_forward(H, 32, q, k, v, mask, flags=ONE | _lib.FLAG_SYNC)
    assert torch.equal(y, y2) and torch.isfinite(y).all()
    if H == 128:
        for flags in (PAIR, 0):
            yp = fa.attention_forward(H, 32, q, k, v, mask, flags=flags | _lib.FLAG_SYNC | _lib.FLAG_NO_SPLIT)
            assert torch.equal(yp, y), flags
    qf, kf, vf = (t.float().view(B, L, R, H).transpose(1, 2) for t in (q, k, v))
    ref = (torch.softmax(qf @ kf.mT / H ** 0.5 + mask.float()[:, None], -1) @ vf).transpose(1, 2).reshape(B, L, R * H)
    d = (y.float() - ref).abs()
    assert float(d.max()) <= MAX_ABS_TOL and float(d.mean()) <= MEAN_ABS_TOL, (float(d.max()), float(d.mean()))


def test_value_of_ones_gives_ones_at_full_size():
    w = WORKLOADS["llama7b_prefill"]
    q, k, _ = workload_inputs(w)
    v = torch.ones_like(q)
    y = run(q, k, v, w.H)
    assert float((y - 1.0).abs().max()) <= 1e-3


def test_linearity_in_values_at_full_size():
    w = WORKLOADS["llama7b_prefill"]
    q, k, v1 = workload_inputs(w)
    v2 = make_inputs(w.B, w.L, w.F, w.sigma, 999)[0]
    dq, dk = q.cuda(), k.cuda()
    f = lambda v: fa.attention_forward(w.H, 128, dq, dk, v.cuda()).float()
    lhs = f((v1.float() * 0.5 + v2.float() * 0.25).half())
    rhs = 0.5 * f(v1) + 0.25 * f(v2)
    torch.cuda.synchronize()
    assert float((lhs - rhs).abs().max()) <= 1e-3


def test_key_permutation_invariance_at_full_size():
    w = WORKLOADS["long_context"]
    q, k, v = workload_inputs(w, heads=slice(0, 8))
    perm = torch.randperm(w.L, generator=torch.Generator().manual_seed(3))
    a = run(q, k, v, w.H)
    b = run(q, k[:, perm].contiguous(), v[:, perm].contiguous(), w.H)
    assert float((a - b).abs().max()) <= 5e-4


def test_host_buffer_entry_point_matches_device_entry_point():
    """The host entry point cuts the call into chunks and runs every chunk with whole work items, so it
    gives the bits of a device-pointer call with FA_B200_FLAG_NO_SPLIT."""
    run = lambda *a, **kw: globals()["run"](*a, flags=WHOLE, **kw)
    q, k, v = make_inputs(2, 300, 256, 1.0, 21)
    y_dev = run(q, k, v, 128)
    y_host = fa.attention_forward_host(128, 128, q.pin_memory(), k.pin_memory(), v.pin_memory()).float()
    assert torch.equal(y_dev, y_host)
    mask = torch.zeros(2, 300, 300, dtype=torch.float16)
    mask[:, :, 250:] = float("-inf")
    y_host_m = fa.attention_forward_host(128, 128, q, k, v, mask).float()
    assert torch.equal(run(q, k, v, 128, mask=mask), y_host_m)
    # B = 1: the chunks are groups of heads moved with pitched copies
    q1, k1, v1 = make_inputs(1, 600, 5 * 128, 1.0, 22)
    assert torch.equal(run(q1, k1, v1, 128), fa.attention_forward_host(128, 128, q1, k1, v1).float())
    m1 = torch.zeros(1, 600, 600, dtype=torch.float16)
    m1[:, :, 500:] = float("-inf")
    assert torch.equal(run(q1, k1, v1, 128, mask=m1), fa.attention_forward_host(128, 128, q1, k1, v1, m1).float())
    # many batch entries: more entries than chunks
    q2, k2, v2 = make_inputs(41, 130, 64, 1.0, 23)
    assert torch.equal(run(q2, k2, v2, 32), fa.attention_forward_host(32, 32, q2, k2, v2).float())
    # large enough to be cut into groups of heads per batch entry (pitched copies), uneven groups, with and without mask
    q3, k3, v3 = make_inputs(2, 1100, 7 * 128, 1.0, 24)
    assert torch.equal(run(q3, k3, v3, 128), fa.attention_forward_host(128, 128, q3, k3, v3).float())
    m3 = torch.zeros(2, 1100, 1100, dtype=torch.float16)
    m3[0, :, 900:] = float("-inf")
    m3[1, :, :100] = float("-inf")
    assert torch.equal(run(q3, k3, v3, 128, mask=m3), fa.attention_forward_host(128, 128, q3, k3, v3, m3).float())
    q4, k4, v4 = make_inputs(1, 2048, 16 * 64, 1.0, 25)
    assert torch.equal(run(q4, k4, v4, 64), fa.attention_forward_host(64, 64, q4, k4, v4).float())


def test_concurrent_callers_from_several_threads():
    """The C ABI is thread-safe: device-pointer calls on separate streams and host-buffer calls
    (which share per-device staging buffers and must serialise themselves) from four threads."""
    import threading
    q, k, v = make_inputs(2, 700, 256, 1.0, 91)
    expected = run(q, k, v, 128)                  # divided schedule, as the device workers below
    expected_whole = run(q, k, v, 128, flags=WHOLE)   # what the host entry point reproduces
    dq, dk, dv = q.cuda(), k.cuda(), v.cuda()
    results, errors = {}, []

    def device_worker(idx):
        try:
            s = torch.cuda.Stream()
            with torch.cuda.stream(s):
                for _ in range(10):
                    y = fa.attention_forward(128, 64, dq, dk, dv)
            s.synchronize()
            results[idx] = y.float().cpu()
        except Exception as exc:  # noqa: BLE001
            errors.append(exc)

    def host_worker(idx):
        try:
            for _ in range(3):
                y = fa.attention_forward_host(128, 64, q, k, v)
            results[idx] = y.float()
        except Exception as exc:  # noqa: BLE001
            errors.append(exc)

    threads = [threading.Thread(target=device_worker, args=(0,)), threading.Thread(target=device_worker, args=(1,)),
               threading.Thread(target=host_worker, args=(2,)), threading.Thread(target=host_worker, args=(3,))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for idx in range(4):
        assert torch.equal(results[idx], expected if idx < 2 else expected_whole)


def test_non_default_stream_and_output_placement():
    q, k, v = (t.cuda() for t in make_inputs(1, 512, 256, 1.0, 31))
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        y = fa.attention_forward(128, 64, q, k, v)
    s.synchronize()
    assert y.device == q.device and y.dtype == torch.float16 and y.shape == q.shape
    assert torch.equal(y, fa.attention_forward(128, 64, q, k, v))


@pytest.mark.parametrize("H,L,R", [(64, 256, 4), (128, 1000, 3)])
def test_operator_can_be_recorded_in_a_cuda_graph(H, L, R):
    """After one ordinary call on the device (which does the once-per-device set-up), a call neither
    allocates nor synchronises: it can be recorded in a CUDA graph and replayed on new input values."""
    q, k, v = (t.cuda() for t in make_inputs(2, L, R * H, 1.0, 31))
    fa.attention_forward(H, 32, q, k, v)                    # set-up outside the recording
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y = fa.attention_forward(H, 32, q, k, v)
    q2, k2, v2 = make_inputs(2, L, R * H, 1.0, 32)
    for dst, src in ((q, q2), (k, k2), (v, v2)):
        dst.copy_(src)
    graph.replay()
    torch.cuda.synchronize()
    assert_close(y.float().cpu(), oracle(q2, k2, v2, H))
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(y, fa.attention_forward(H, 32, q, k, v))


def test_error_behaviour_on_gpu_tensors():
    q, k, v = (t.cuda() for t in make_inputs(1, 64, 128, 1.0, 41))
    with pytest.raises(RuntimeError):
        fa.attention_forward(48, 32, q, k, v)                 # head_dim not a power of two
    with pytest.raises(RuntimeError):
        fa.attention_forward(128, 16, q, k, v)                # forbidden pair
    with pytest.raises(RuntimeError):
        fa.attention_forward(64, 64, q, k[:, :32].contiguous(), v)
    with pytest.raises(RuntimeError):
        fa.attention_forward(64, 64, q.float(), k.float(), v.float())
    with pytest.raises(RuntimeError):
        fa.attention_forward(64, 64, q.transpose(1, 2), k, v)  # not contiguous


def test_bounded_wait_gives_up_and_reports_without_harming_the_gpu():
    out = (ctypes.c_uint32 * 3)()
    assert _lib.load().fa_b200_selftest_bounded_wait(0, out) == 0
    assert (out[0], out[1], out[2]) == (0x67F, 1, 2)
    # the context is still usable
    q, k, v = make_inputs(1, 128, 64, 1.0, 51)
    assert_close(run(q, k, v, 64), oracle(q, k, v, 64))


def test_more_batch_entries_than_a_grid_axis_holds():
    """70000 one-tile problems: the reference puts the batch on the x axis of its grid
    (include/fused_attn.cuh:883) and takes such a shape; so does this launcher."""
    B, L, H = 70000, 8, 16
    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    q, k, v = (torch.randn(B, L, H, generator=g, device="cuda", dtype=torch.float16) for _ in range(3))
    y = fa.attention_forward(H, 16, q, k, v, flags=_lib.FLAG_SYNC)
    ref = torch.softmax(q.float() @ k.float().mT / H ** 0.5, -1) @ v.float()
    d = (y.float() - ref).abs()
    assert float(d.max()) <= MAX_ABS_TOL and float(d.mean()) <= MEAN_ABS_TOL


# ---------------------------------------------------------------- the checked build
def _checked_lib():
    path = os.path.join(os.path.dirname(fa.__file__), "lib", "libfa_b200_debug.so")
    if not os.path.exists(path):
        pytest.skip("checked library not built (python -m fused_attention_b200.build --debug)")
    lib = ctypes.CDLL(path)
    u32, vp, i32 = ctypes.c_uint32, ctypes.c_void_p, ctypes.c_int
    lib.fa_b200_attention_forward.restype = i32
    lib.fa_b200_attention_forward.argtypes = [vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, i32, vp, u32]
    lib.fa_b200_read_status.restype = i32
    lib.fa_b200_read_status.argtypes = [i32, ctypes.POINTER(u32)]
    lib.fa_b200_selftest_debug_checks.restype = i32
    lib.fa_b200_selftest_debug_checks.argtypes = [i32, ctypes.POINTER(u32)]
    return lib


def test_checked_build_refuses_bad_operands_without_touching_memory():
    """The predicates of the checked build (-DFA_DEBUG), asked about operands that are in order and operands
    that are not; no copy is made.  The normal library has no checks and says so."""
    out = (ctypes.c_uint32 * 4)()
    assert _checked_lib().fa_b200_selftest_debug_checks(0, out) == 0
    assert (out[0], out[1], out[2], out[3]) == (0x703, 1, 1, 0x7FF)
    assert _lib.load().fa_b200_selftest_debug_checks(0, out) == 0 and out[2] == 0


@pytest.mark.parametrize("H,B,R,L,flags,masked", [
    (16, 2, 3, 200, SIMPLE, False), (64, 2, 3, 300, SIMPLE, True), (64, 3, 5, 700, ONE, False), (64, 2, 2, 520, ONE, True),
    (128, 2, 3, 1000, ONE, False), (128, 2, 4, 2048, PAIR, False), (128, 1, 4, 2048 + 77, 0, False), (128, 1, 2, 650, ONE, True),
    (128, 20, 10, 300, PAIR, False), (128, 2, 3, 1000, PAIR, True), (128, 3, 4, 2048, PAIR, True)])
def test_checked_build_runs_clean_and_gives_the_same_bits(H, B, R, L, flags, masked):
    """Every kernel under the checked build: each TMA copy and tensor-memory access is checked against the
    CTA's tile area, the tensor's extent and the CTA's tensor-memory allocation, tile buffers and Y are
    filled with NaN beforehand.  No check may fire, no NaN may survive, and the bits are the normal build's."""
    lib = _checked_lib()
    g = torch.Generator(device="cuda")
    g.manual_seed(L + H)
    q, k, v = (torch.randn(B, L, R * H, generator=g, device="cuda").half() for _ in range(3))
    mask = None
    if masked:
        mask = torch.triu(torch.full((L, L), float("-inf"), device="cuda", dtype=torch.float16), diagonal=1)
        mask = mask.unsqueeze(0).expand(B, L, L).contiguous()
    y = torch.empty_like(q)
    rc = lib.fa_b200_attention_forward(q.data_ptr(), k.data_ptr(), v.data_ptr(), None if mask is None else mask.data_ptr(),
                                       y.data_ptr(), B, L, R * H, H, 0, 0, None, flags | _lib.FLAG_SYNC)
    assert rc == 0, rc
    w = (ctypes.c_uint32 * 2)()
    assert lib.fa_b200_read_status(0, w) == 0 and (w[0], w[1]) == (0, 0), hex(w[0])
    assert torch.isfinite(y).all()
    assert torch.equal(y, fa.attention_forward(H, 16 if H < 128 else 32, q, k, v, mask, flags=flags | _lib.FLAG_SYNC))


@pytest.mark.parametrize("flags", [ONE, PAIR])
def test_clock_counting_build_reports_a_launch(flags):
    """The -DFA_CYCLES build (fused_attention_b200/cycles.py): CTA 0's time stamps are in order, its busy time is
    most of the period of back-to-back launches, and its SM clock count over that time is a clock a B200 can run at."""
    from fused_attention_b200 import build, cycles
    if not os.path.exists(build.CYCLES_LIB):
        pytest.skip("clock-counting library not built (python -m fused_attention_b200.build --cycles)")
    s = cycles.measure(2, 16, 2048, 128, flags=flags, launches=30)
    assert s["launches"] >= 20, s
    assert 0.5 * s["period_us"] <= s["busy_us"] <= s["period_us"], s
    mhz = s["sm_clocks"] / s["busy_us"]
    assert 900.0 <= mhz <= 2100.0, (mhz, s)


def test_time_line_build_reports_the_key_step():
    """The -DFA_CYCLES -DFA_TIMELINE build: the stamps of one launch of the kernel on pairs of CTAs give a key step
    of a few thousand SM clocks, a softmax pass that fits into it, and waits that are shorter than the step."""
    from fused_attention_b200 import build, cycles
    if not os.path.exists(build.TIMELINE_LIB):
        pytest.skip("time-line library not built (python -m fused_attention_b200.build --cycles)")
    r = cycles.timeline(2, 16, 4096, 128)      # 32 key steps per item, several items per pair of CTAs
    assert r["steps_recorded"] >= 64, r
    assert 1800.0 <= r["step_period"] <= 5000.0, r
    for tile in ("tile0", "tile1"):
        assert 1000.0 <= r[tile]["pass"] <= r["step_period"] * 1.05, r
        assert 0.0 <= r[tile]["wait_for_S"] <= r["step_period"], r
    assert r["qk_warp"]["wait_for_S_read_by_tile0"] <= r["step_period"], r


# ---------------------------------------------------------------- drop-in module `fused_attn`
def _fused_attn_module():
    ext_dir = os.path.join(os.path.dirname(fa.__file__), "ext")
    if ext_dir not in sys.path:
        sys.path.insert(0, ext_dir)
    import fused_attn
    return fused_attn


@pytest.mark.parametrize("H,C", [(16, 16), (16, 32), (32, 16), (32, 32), (32, 64), (64, 16), (64, 32), (64, 64),
                                 (64, 128), (128, 32), (128, 64), (128, 128)])
def test_reference_unit_tests_through_the_torch_extension(H, C):
    """The reference's own twelve cases (tests/test_fused_attn.py:12-67): B=1, R=2, L=2*C, N(0,1)
    inputs drawn on the GPU with seed 179, compared at its tolerance rtol=atol=1e-2."""
    fused_attn = _fused_attn_module()
    torch.random.manual_seed(179)
    q, k, v = (torch.randn(1, 2 * C, 2 * H, device="cuda", dtype=torch.float16) for _ in range(3))
    expected = oracle(q.cpu(), k.cpu(), v.cpu(), H)
    actual = fused_attn.attention_forward(H, C, q, k, v)
    assert actual.dtype == torch.float16 and actual.device == q.device
    torch.testing.assert_close(actual.float().cpu(), expected, rtol=0.01, atol=0.01)
    assert_close(actual.float().cpu(), expected)


def test_torch_extension_accepts_mask_keyword_and_ragged_length():
    fused_attn = _fused_attn_module()
    q, k, v = (t.cuda() for t in make_inputs(2, 197, 128, 1.0, 61))
    mask = torch.zeros(2, 197, 197, dtype=torch.float16, device="cuda")
    mask[:, :, 150:] = float("-inf")
    y = fused_attn.attention_forward(head_dim=64, chunk_size=64, queries=q, keys=k, values=v, mask=mask)
    assert_close(y.float().cpu(), oracle(q.cpu(), k.cpu(), v.cpu(), 64, mask.cpu()))


# ---------------------------------------------------------------- the reference's own CUDA kernel
def _ref_wmma():
    path = os.path.join(os.path.dirname(os.path.dirname(__file__)), "oracle", "_ref", "libref_fused_attn.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref not built (needs the reference checkout at build time)")
    lib = ctypes.CDLL(path)
    lib.ref_wmma_attention_forward.restype = ctypes.c_int
    lib.ref_wmma_attention_forward.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_uint32] * 5
    return lib


def _run_ref_wmma(lib, q, k, v, H, C, mask=None):
    B, L, F = q.shape
    y_ref = torch.empty_like(q)
    assert lib.ref_wmma_attention_forward(q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                          None if mask is None else mask.data_ptr(), y_ref.data_ptr(),
                                          B, L, F, H, C) == 0
    torch.cuda.synchronize()
    return y_ref


@pytest.mark.parametrize("H,C", [(16, 16), (16, 32), (32, 16), (32, 32), (32, 64), (64, 16), (64, 32), (64, 64),
                                 (64, 128), (128, 32), (128, 64), (128, 128)])
def test_against_the_reference_fused_kernel_on_its_own_test_shapes(H, C):
    """The reference's WMMA kernel (compiled for sm_100a from its own header) on the shapes its
    unit tests use (B=1, R=2, L=2*C).  Where the reference kernel itself is within 5e-3 of the fp32
    oracle the two kernels must agree at the reference's tolerance rtol=atol=1e-2; where it is not
    (its fp16 accumulation and its unsynchronised shared-memory alias make some instances drift on
    this GPU) this implementation must still be the closer one."""
    lib = _ref_wmma()
    hq, hk, hv = make_inputs(1, 2 * C, 2 * H, 1.0, 179)
    q, k, v = hq.cuda(), hk.cuda(), hv.cuda()
    expected = oracle(hq, hk, hv, H)
    y_ref = _run_ref_wmma(lib, q, k, v, H, C)
    y = fa.attention_forward(H, C, q, k, v)
    err_new = assert_close(y.float().cpu(), expected)
    err_ref = error_metrics(y_ref.float().cpu(), expected)
    if err_ref["max_abs"] <= 5e-3:
        torch.testing.assert_close(y.float(), y_ref.float(), rtol=0.01, atol=0.01)
    assert err_new["max_abs"] <= err_ref["max_abs"], (err_new, err_ref)


@pytest.mark.parametrize("H,C", [(64, 64), (64, 128), (128, 128), (32, 32), (16, 32), (128, 64)])
def test_mask_against_the_reference_kernel_single_chunk(H, C):
    """The mask semantics pinned to the reference itself.  Its kernel adds the mask tile only while it
    works on the first key chunk (include/fused_attn.cuh:732-742), so with L == chunk_size, where the
    first chunk is the whole key axis, it is a valid oracle for what the mask means: an additive
    [B, L, L] array shared by all heads (include/fused_attn.cuh:686, 738).  Causal and padding masks
    with soft values in between, no row masked out completely; the two kernels must agree at the
    reference's rtol = atol = 1e-2 and this one must meet the fp32 oracle's bounds."""
    lib = _ref_wmma()
    B, R, L = 2, 2, C
    hq, hk, hv = make_inputs(B, L, R * H, 1.0, 900 + H + C)
    mask = torch.zeros(B, L, L, dtype=torch.float16)
    mask[0] = torch.triu(torch.full((L, L), float("-inf")), diagonal=1).half()          # causal
    mask[1, :, L - L // 4:] = float("-inf")                                               # padding
    mask[1, :, : L // 2] += 0.5 * torch.randn(L, L // 2, generator=torch.Generator().manual_seed(C)).half()
    q, k, v, dmask = hq.cuda(), hk.cuda(), hv.cuda(), mask.cuda()
    expected = oracle(hq, hk, hv, H, mask)
    y_ref = _run_ref_wmma(lib, q, k, v, H, C, dmask)
    err_ref = error_metrics(y_ref.float().cpu(), expected)
    assert err_ref["max_abs"] <= 1e-2, err_ref       # the reference kernel and the oracle formula mean the same mask
    for flags in kernels_for(H):
        y = fa.attention_forward(H, C, q, k, v, dmask, flags=flags | _lib.FLAG_SYNC)
        torch.testing.assert_close(y.float(), y_ref.float(), rtol=0.01, atol=0.01)
        assert_close(y.float().cpu(), expected)


@pytest.mark.parametrize("H,C,B,R,L", [(64, 64, 1, 4, 256), (128, 128, 2, 4, 512), (64, 128, 8, 12, 512)])
def test_closer_to_the_oracle_than_the_reference_fused_kernel(H, C, B, R, L):
    """Beyond two key chunks the reference kernel (all-fp16 arithmetic, and a shared-memory alias
    that lets warps overwrite scores other warps still read, include/fused_attn.cuh:659,677,822-831)
    drifts from the fp32 oracle; this implementation must not, and must be at least as close."""
    lib = _ref_wmma()
    hq, hk, hv = make_inputs(B, L, R * H, 1.0, 71)
    q, k, v = hq.cuda(), hk.cuda(), hv.cuda()
    expected = oracle(hq, hk, hv, H)
    err_ref = error_metrics(_run_ref_wmma(lib, q, k, v, H, C).float().cpu(), expected)
    err_new = assert_close(fa.attention_forward(H, C, q, k, v).float().cpu(), expected)
    assert err_new["max_abs"] <= err_ref["max_abs"] and err_new["mean_abs"] <= err_ref["mean_abs"], (err_new, err_ref)


# ---------------------------------------------------------------- torch-free C++ driver
@pytest.mark.parametrize("shape", [(2, 4, 600, 128), (3, 2, 197, 64), (1, 2, 100, 32)])
def test_torch_free_driver_program(shape):
    """The C++ program over the C ABI (the role of the reference's src/test.cu): fills with an LCG,
    runs both entry points, checks sampled rows against a plain CPU loop and exits non-zero on a miss."""
    import subprocess
    from fused_attention_b200 import build
    exe = build.driver_path()
    if not os.path.exists(exe):
        pytest.skip("driver not built (python -m fused_attention_b200.build --driver)")
    r = subprocess.run([exe, *map(str, shape), "5"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "differ in 0 values" in r.stdout


def test_bound_call_is_the_same_launch():
    """bind_forward checks and converts the arguments once; its launch() writes the same bits into `out` as
    attention_forward returns, call after call, and rejects what attention_forward rejects."""
    q, k, v = (t.cuda() for t in make_inputs(2, 700, 3 * 128, 1.0, 77))
    out = torch.zeros_like(q)
    launch, y = fa.bind_forward(128, 64, q, k, v, out=out)
    assert y is out
    for _ in range(3):
        out.zero_()
        launch()
        torch.cuda.synchronize()
        assert torch.equal(out, fa.attention_forward(128, 64, q, k, v))
    with pytest.raises(Exception):
        fa.bind_forward(128, 64, q, k[:, :10], v)
