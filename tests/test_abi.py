"""The C ABI without a GPU: the library loads, exports what the header declares, and rejects bad
arguments with the documented codes before touching CUDA."""
import ctypes
import os
import re

import pytest

from fused_attention_b200 import _lib


@pytest.fixture(scope="module")
def lib():
    return _lib.load()


def _header(repo_root):
    with open(os.path.join(repo_root, "include", "fa_b200.h")) as f:
        return f.read()


def test_library_exports_every_declared_symbol(lib, repo_root):
    text = _header(repo_root)
    # what the header declares only for a variant build (#ifdef FA_CYCLES ... #endif) is that variant's
    variant = "".join(re.findall(r"#ifdef FA_CYCLES\n(.*?)#endif", text, flags=re.S))
    only_variant = set(re.findall(r"\b(fa_b200_\w+)\s*\(", variant))
    declared = set(re.findall(r"\b(fa_b200_\w+)\s*\(", text)) - only_variant
    assert declared == set(_lib.EXPORTED_SYMBOLS)
    for name in declared:
        assert getattr(lib, name) is not None
    assert only_variant == {"fa_b200_debug_cycles"}
    from fused_attention_b200 import build
    if os.path.exists(build.CYCLES_LIB):
        import ctypes
        for path in (build.CYCLES_LIB, build.TIMELINE_LIB):
            if os.path.exists(path):
                variant_lib = ctypes.CDLL(path)
                for name in declared | only_variant:
                    assert getattr(variant_lib, name) is not None


def test_python_constants_match_header(repo_root):
    text = _header(repo_root)
    for cname, value in re.findall(r"(FA_B200_(?:ERR_\w+|OK|FLAG_\w+))\s*=\s*(-?\d+)u?", text):
        py = cname.replace("FA_B200_", "")
        assert getattr(_lib, py) == int(value), cname


def test_strerror_covers_all_codes(lib):
    seen = set()
    for code in range(0, -11, -1):
        s = _lib.strerror(code)
        assert s and s != _lib.strerror(-99)
        seen.add(s)
    assert len(seen) == 11
    assert "unknown" in _lib.strerror(-99)


A16 = ctypes.create_string_buffer(64)


def _aligned():
    base = ctypes.addressof(A16)
    return (base + 15) & ~15


def _call(lib, q=None, k=None, v=None, mask=None, y=None, B=1, L=32, F=64, H=32, chunk=32, flags=0):
    a = _aligned()
    q = a if q is None else q
    k = a if k is None else k
    v = a if v is None else v
    y = a if y is None else y
    return lib.fa_b200_attention_forward(q, k, v, mask, y, B, L, F, H, chunk, 0, None, flags)


def test_argument_rejections_happen_before_any_cuda_call(lib):
    assert _call(lib, q=0) == _lib.ERR_NULL_POINTER
    assert _call(lib, y=0) == _lib.ERR_NULL_POINTER
    for H in (0, 8, 24, 48, 256):
        assert _call(lib, H=H, F=H * 2 if H else 64) == _lib.ERR_HEAD_DIM
    # reference rule set for chunk_size, src/fused_attn_extention.cu:46-47
    assert _call(lib, H=32, chunk=128) == _lib.ERR_CHUNK      # > 2*head_dim
    assert _call(lib, H=32, chunk=24) == _lib.ERR_CHUNK       # not a power of two
    assert _call(lib, H=32, chunk=8) == _lib.ERR_CHUNK        # < 16
    assert _call(lib, H=128, F=128, chunk=16) == _lib.ERR_CHUNK
    assert _call(lib, H=64, F=128, chunk=256) == _lib.ERR_CHUNK
    assert _call(lib, B=0) == _lib.ERR_SHAPE
    assert _call(lib, L=0) == _lib.ERR_SHAPE
    assert _call(lib, F=48, H=32) == _lib.ERR_SHAPE
    assert _call(lib, q=_aligned() + 2) == _lib.ERR_ALIGNMENT
    assert _call(lib, flags=3) == _lib.ERR_FLAGS               # both force bits
    assert _call(lib, flags=1024) == _lib.ERR_FLAGS            # unknown bit
    assert _call(lib, flags=_lib.FLAG_NO_OVERLAP | 3) == _lib.ERR_FLAGS
    assert _call(lib, B=0, flags=_lib.FLAG_NO_OVERLAP) == _lib.ERR_SHAPE   # the bit itself is known
    assert _call(lib, H=32, flags=_lib.FLAG_FORCE_PIPELINED) == _lib.ERR_FLAGS
    assert _call(lib, H=64, F=64, flags=_lib.FLAG_FORCE_PAIR) == _lib.ERR_FLAGS              # head_dim 128 only
    assert _call(lib, H=128, F=128, flags=_lib.FLAG_FORCE_PAIR | _lib.FLAG_NO_PAIR) == _lib.ERR_FLAGS
    # with a mask only when TMA can fetch its tiles: every mask row on a 16-byte boundary
    assert _call(lib, H=128, F=128, mask=_aligned() + 2, flags=_lib.FLAG_FORCE_PAIR) == _lib.ERR_FLAGS
    assert _call(lib, H=128, F=128, L=36, mask=_aligned(), flags=_lib.FLAG_FORCE_PAIR) == _lib.ERR_FLAGS


def test_host_entry_rejections(lib):
    a = _aligned()
    f = lib.fa_b200_attention_forward_host
    assert f(0, a, a, None, a, 1, 32, 64, 32, 32, 0, 0) == _lib.ERR_NULL_POINTER
    assert f(a, a, a, None, a, 1, 32, 64, 12, 32, 0, 0) == _lib.ERR_HEAD_DIM
    assert f(a + 2, a, a, None, a, 1, 32, 60, 32, 32, 0, 0) == _lib.ERR_SHAPE  # host pointers may be unaligned


def test_kernel_selection(lib):
    sel = lib.fa_b200_select_kernel
    assert sel(4, 2048, 4096, 128, 0, 0) == 3      # headline: pipelined, on pairs of CTAs
    assert sel(4, 2048, 4096, 128, 0, _lib.FLAG_NO_PAIR) == 2
    assert sel(4, 2048, 4096, 128, 1, 0) == 3      # with a mask too, its rows being 16-byte aligned
    assert sel(4, 2048, 512, 128, 0, 0) == 2       # 64 blocks of 512 rows for 74 pairs of SMs: single CTAs
    assert sel(4, 2048, 512, 128, 1, 0) == 3       # ... but pairs with a mask (a mask buffer per query tile)
    assert sel(4, 2048, 1024, 128, 0, 0) == 3      # 128 blocks: two rounds of pairs
    assert sel(4, 2044, 4096, 128, 1, 0) == 2      # mask rows that TMA cannot fetch: single CTAs
    assert sel(1, 16384, 4096, 128, 0, 0) == 3
    assert sel(1, 16384, 512, 128, 0, 0) == 2      # the last round of this one is divided: single CTAs
    assert sel(4, 2048 + 256, 4096, 128, 0, 0) == 2    # nine 256-row blocks: an odd one would idle half a pair
    assert sel(1, 256, 256, 64, 0, 0) == 1         # tiny: simple
    assert sel(64, 197, 1024, 64, 0, 0) == 2       # 1024 items of two key steps: persistent kernel
    assert sel(64, 100, 1024, 64, 0, 0) == 1       # a single partial tile per (batch, head)
    assert sel(1, 2048, 512, 128, 0, 0) == 2       # 32 items only, but 16 key steps each: pipelined (divided)
    assert sel(1, 512, 512, 128, 0, 0) == 1        # 8 items of 4 key steps cannot occupy the SMs
    assert sel(4, 2048, 512, 16, 0, 0) == 1        # small head_dim
    assert sel(4, 2048, 512, 32, 1, 0) == 1
    assert sel(4, 2048, 4096, 128, 0, _lib.FLAG_FORCE_SIMPLE) == 1
    assert sel(1, 256, 256, 64, 0, _lib.FLAG_FORCE_PIPELINED) == 2
    assert sel(1, 256, 250, 64, 0, 0) == _lib.ERR_SHAPE
    # no limit of 65535 on batch entries or heads (the reference has none on its batch axis)
    assert sel(70000, 64, 64, 64, 0, 0) == 1
    assert sel(1, 64, 70000 * 16, 16, 0, 0) == 1
    assert sel(1 << 20, 128 * 2048, 64, 64, 0, 0) == _lib.ERR_SHAPE   # 2^31 CTAs: too many for one grid axis


def test_missing_library_is_loud(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(_lib.LibraryNotBuilt):
        _lib.load()
