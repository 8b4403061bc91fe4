"""The entry point for callers that cannot allocate device memory.

`fa_b200_attention_forward_noalloc` is for code that must not call cudaMalloc: a process whose
device memory belongs entirely to another allocator or is already handed out, a loop where an
allocation would synchronise the device, a plugin that is not allowed to grow the footprint of its
host.  Its kernel's scratch (one status pair per CTA) sits in a fixed 128 KiB array inside the
library instead of in allocated memory, which caps the problem at 16384 CTAs and makes all calls on
a device share that array.

This file is collected last on purpose: if it fails, `pytest -x` has already run everything else.
It must pass alone in a fresh process and after the rest of the suite, so it makes no assumption
about which entry points ran before it.
"""
import ctypes

import pytest
import torch

from fused_attention_b200 import _lib
from fused_attention_b200.workloads import make_inputs
from oracle.naive_attention import MAX_ABS_TOL, MEAN_ABS_TOL, attention as oracle, error_metrics

pytestmark = pytest.mark.gpu


def _device_tensors(B, L, F, seed):
    q, k, v = (t.cuda() for t in make_inputs(B, L, F, 1.0, seed))
    torch.cuda.synchronize()
    return q, k, v


def _existing(lib, q, k, v, H, mask=None):
    """Reference result: the established entry point, forced onto the same one-tile-per-CTA kernel."""
    B, L, F = q.shape
    y = torch.empty_like(q)
    rc = lib.fa_b200_attention_forward(q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                       None if mask is None else mask.data_ptr(), y.data_ptr(),
                                       B, L, F, H, 0, 0, None, _lib.FLAG_FORCE_SIMPLE | _lib.FLAG_SYNC)
    assert rc == 0, _lib.strerror(rc)
    return y


def _noalloc(lib, q, k, v, H, y, mask=None):
    B, L, F = q.shape
    return lib.fa_b200_attention_forward_noalloc(q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                                 None if mask is None else mask.data_ptr(), y.data_ptr(),
                                                 B, L, F, H, 0, 0, None, _lib.FLAG_SYNC)


@pytest.mark.parametrize("H,B,R,L", [(128, 2, 3, 300), (64, 1, 4, 197), (16, 2, 2, 70)])
def test_two_calls_in_a_row_match_the_existing_entry_point(H, B, R, L):
    lib = _lib.load()
    q, k, v = _device_tensors(B, L, R * H, 500 + L)
    expected = _existing(lib, q, k, v, H)
    # the outputs are allocated by the caller, here; the call itself allocates nothing
    y1 = torch.full_like(q, float("nan"))
    y2 = torch.full_like(q, float("nan"))
    assert _noalloc(lib, q, k, v, H, y1) == 0
    assert _noalloc(lib, q, k, v, H, y2) == 0      # second call reuses the shared scratch array
    # same kernel arithmetic on the same inputs: identical bits, well inside the suite's
    # tolerance of max-abs 2e-3 / mean-abs 2e-4
    assert torch.equal(y1, expected)
    assert torch.equal(y2, expected)
    # and against the CPU oracle on the same inputs, with the suite's bounds
    m = error_metrics(y2.float().cpu(), oracle(q.cpu(), k.cpu(), v.cpu(), H))
    assert m["max_abs"] <= MAX_ABS_TOL and m["mean_abs"] <= MEAN_ABS_TOL, m
    # calls after the first leave the device's memory as it was
    free_before = torch.cuda.mem_get_info()[0]
    assert _noalloc(lib, q, k, v, H, y1) == 0
    assert torch.cuda.mem_get_info()[0] == free_before


def test_second_call_with_other_shape_and_mask_after_the_first():
    lib = _lib.load()
    q, k, v = _device_tensors(1, 260, 128, 77)
    y = torch.empty_like(q)
    assert _noalloc(lib, q, k, v, 64, y) == 0
    assert torch.equal(y, _existing(lib, q, k, v, 64))
    # a different grid right after: its status pairs were cleared by the call itself
    q2, k2, v2 = _device_tensors(2, 130, 64, 78)
    mask = torch.zeros(2, 130, 130, dtype=torch.float16, device="cuda")
    mask[:, :, 100:] = float("-inf")
    y2 = torch.empty_like(q2)
    assert _noalloc(lib, q2, k2, v2, 32, y2, mask) == 0
    assert torch.equal(y2, _existing(lib, q2, k2, v2, 32, mask))


def test_the_largest_grid_the_scratch_holds_runs_and_a_smaller_one_after_it():
    """Exactly 16384 CTAs (16 query tiles x 32 heads x 32 batch entries) use every status pair of the
    array; the call after it has a small grid and must not be disturbed by what the large one left."""
    lib = _lib.load()
    H, B, R, L = 16, 32, 32, 2048
    g = torch.Generator(device="cuda")
    g.manual_seed(9)
    q, k, v = (torch.randn(B, L, R * H, generator=g, device="cuda", dtype=torch.float16) for _ in range(3))
    y = torch.empty_like(q)
    assert _noalloc(lib, q, k, v, H, y) == 0
    assert torch.equal(y, _existing(lib, q, k, v, H))
    for b, h in ((0, 0), (B - 1, R - 1)):
        qf, kf, vf = (t[b, :, h * H:(h + 1) * H].float() for t in (q, k, v))
        d = (y[b, :, h * H:(h + 1) * H].float() - torch.softmax(qf @ kf.T / H ** 0.5, -1) @ vf).abs()
        assert float(d.max()) <= MAX_ABS_TOL and float(d.mean()) <= MEAN_ABS_TOL
    q2, k2, v2 = _device_tensors(1, 100, 32, 79)
    y2 = torch.empty_like(q2)
    assert _noalloc(lib, q2, k2, v2, 16, y2) == 0
    assert torch.equal(y2, _existing(lib, q2, k2, v2, 16))


def test_work_beyond_the_fixed_capacity_is_rejected_before_launch():
    lib = _lib.load()
    a = ctypes.create_string_buffer(64)
    p = (ctypes.addressof(a) + 15) & ~15          # aligned dummy: the call must return before using it
    # 16 * 33 * 32 = 16896 CTAs > 16384
    rc = lib.fa_b200_attention_forward_noalloc(p, p, p, None, p, 32, 2048, 33 * 64, 64, 0, 0, None, 0)
    assert rc == _lib.ERR_TOO_LARGE
    assert "capacity" in _lib.strerror(rc)
    # flags other than SYNC make no sense for a single-kernel entry point
    rc = lib.fa_b200_attention_forward_noalloc(p, p, p, None, p, 1, 128, 64, 64, 0, 0, None,
                                               _lib.FLAG_FORCE_PIPELINED)
    assert rc == _lib.ERR_FLAGS
