"""The C-ABI library without a GPU: it loads, exports every symbol the header
declares, answers the host-only queries, and its tile schedule covers every unit of
work exactly once."""

import ctypes
import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]


def _declared_symbols():
    text = (ROOT / "include" / "chord_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(chord_b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(native_lib):
    from chord_b200 import _lib

    declared = _declared_symbols()
    assert len(declared) >= 15
    for name in declared:
        assert hasattr(native_lib, name), f"{name} is declared in include/chord_b200.h but not exported"
    # and the Python binding knows each of them
    assert sorted(_lib.SIGNATURES) == declared


def test_version_and_error_channel(native_lib):
    from chord_b200 import _lib

    assert native_lib.chord_b200_version().startswith(b"chord_b200")
    assert native_lib.chord_b200_set_option(b"no_such_option", 1) == 1
    assert "no_such_option" in _lib.last_error()
    with pytest.raises(ValueError):
        _lib.set_option("dequant_groups", 3)
    _lib.set_option("dequant_groups", 2)


def test_block_m_queries(native_lib):
    for routed in (0, 1, 8, 160, 400, 2048, 4096, 32768, 10**6):
        for n, k, e in ((4096, 7168, 48), (7168, 2048, 48), (1024, 512, 8), (4096, 7168, 384)):
            bm = native_lib.chord_b200_indexed_block_m(n, k, e, routed)
            assert bm % 8 == 0 and 8 <= bm <= 256
    # more rows per expert never shrink the block
    prev = 0
    for routed in range(0, 48 * 300, 48):
        bm = native_lib.chord_b200_indexed_block_m(4096, 7168, 48, routed)
        assert bm >= prev
        prev = bm
    assert [native_lib.chord_b200_masked_tile_m(m) for m in (1, 8, 9, 20, 21, 48, 49, 144, 145, 10**4)] == \
        [16, 16, 32, 32, 64, 64, 128, 128, 256, 256]


def _segments(lib, tiles, k, grid, cta):
    cap = 8192
    buf = (ctypes.c_int32 * (5 * cap))()
    n = lib.chord_b200_schedule_segments(tiles, k, grid, cta, ctypes.cast(buf, ctypes.c_void_p), cap)
    assert 0 <= n <= cap
    return np.frombuffer(buf, dtype=np.int32)[: 5 * n].reshape(n, 5).copy()


@pytest.mark.parametrize("tiles,k,grid", [
    (0, 512, 148), (1, 128, 148), (1, 7168, 148), (5, 2048, 148), (32, 7168, 148),
    (147, 2048, 148), (148, 2048, 148), (149, 7168, 148), (352, 7168, 148), (300, 512, 148),
    (1536, 7168, 148), (2688, 2048, 148), (37, 2368, 16), (1000, 64, 7),
])
def test_schedule_covers_every_unit_once(native_lib, tiles, k, grid):
    k_iters = (k + 127) // 128
    cover = np.zeros((tiles, k_iters), dtype=np.int64)
    owners, contributors = {}, {}
    for cta in range(grid):
        segs = _segments(native_lib, tiles, k, grid, cta)
        seen_partial_contrib = 0
        for tile, kb, ke, kind, peer in segs:
            assert 0 <= tile < tiles and 0 <= kb < ke <= k_iters
            cover[tile, kb:ke] += 1
            if kind == 0:
                assert kb == 0 and ke == k_iters
            elif kind == 1:
                assert kb == 0 and ke < k_iters and peer >= 1
                assert tile not in owners
                owners[tile] = (cta, peer)
            else:
                assert kind == 2 and kb > 0 and peer < cta
                contributors.setdefault(tile, []).append((cta, peer))
                seen_partial_contrib += 1
        # one workspace slot and one lock word per CTA are enough
        assert seen_partial_contrib <= 1
        assert sum(1 for s in segs if s[3] == 1) <= 1
    assert (cover == 1).all()
    assert set(owners) == set(contributors)
    for tile, (cta, count) in owners.items():
        ctas = sorted(c for c, _ in contributors[tile])
        assert ctas == list(range(cta + 1, cta + 1 + count))      # summed in CTA order
        assert all(owner == cta for _, owner in contributors[tile])


def test_schedule_owner_never_waits_on_an_earlier_cta(native_lib):
    """Deadlock freedom: an owner's slice is the last work of its CTA and every
    contributor slice is the first stream-K work of a later CTA."""
    tiles, k, grid = 352, 7168, 148
    for cta in range(grid):
        segs = _segments(native_lib, tiles, k, grid, cta)
        kinds = [int(s[3]) for s in segs]
        if 1 in kinds:
            assert kinds.index(1) == len(kinds) - 1
        if 2 in kinds:
            before = kinds[: kinds.index(2)]
            assert all(kind == 0 for kind in before)


@pytest.mark.parametrize("tiles,k,grid", [(32, 7168, 592), (56, 2048, 592), (1, 7168, 592), (3, 512, 148),
                                          (352, 7168, 592), (1088, 7168, 592)])
def test_schedule_slices_are_not_slivers(native_lib, tiles, k, grid):
    """The stream-K tail is cut into slices of at least eight k-blocks (fewer only if the
    whole tail is shorter), also when there are far more workers than work: the decode
    kernel schedules four workers per SM."""
    k_iters = (k + 127) // 128
    lengths, busy = [], 0
    for cta in range(grid):
        segs = _segments(native_lib, tiles, k, grid, cta)
        partial = [(int(ke - kb)) for _, kb, ke, kind, _ in segs if kind != 0]
        whole = [1 for _, _, _, kind, _ in segs if kind == 0]
        if len(segs):
            busy += 1
        work = sum(int(ke - kb) for _, kb, ke, _, _ in segs)
        if work and partial:
            lengths.append(work)
    tail_units = (tiles % grid if tiles >= grid else tiles) * k_iters
    if lengths:
        assert min(lengths) >= min(8, tail_units)
    assert busy <= max(1, grid)


def test_schedule_rejects_bad_queries(native_lib):
    assert native_lib.chord_b200_schedule_segments(10, 100, 148, 0, None, 0) < 0
    assert native_lib.chord_b200_schedule_segments(10, 128, 148, 148, None, 0) < 0
    assert native_lib.chord_b200_schedule_segments(10, 128, 148, 3, None, 0) >= 0


def test_misaligned_pointers_are_refused_before_any_launch(native_lib):
    """The kernels read activations and the SiLU*mul operands in 16-byte pieces: a pointer
    that is not 16-byte aligned comes back as return code 1 from the argument checks (no
    device is touched, so this runs without a GPU)."""
    from chord_b200 import _lib

    ok, odd = 0x7F0000000000, 0x7F0000000008
    lib = native_lib
    assert lib.chord_b200_silu_mul(odd, ok, 4, 64, None) == 1
    assert "aligned" in _lib.last_error()
    assert lib.chord_b200_silu_mul(ok, odd, 4, 64, None) == 1
    assert lib.chord_b200_silu_mul_routed(odd, ok, ok, 16, ok, 4, 64, None) == 1

    def indexed(x, workspace, out):
        return lib.chord_b200_indexed(x, ok, ok, ok, 16, ok, 1, ok, out, ok, 1024, workspace, 1 << 20,
                                      None, 4, 128, 64, 1, 1, 16, None)

    assert indexed(odd, ok, ok) == 1 and "activation" in _lib.last_error()
    assert indexed(ok, odd, ok) == 1 and "workspace" in _lib.last_error()
    assert indexed(ok, ok, odd) == 1 and "output" in _lib.last_error()
    assert lib.chord_b200_masked(odd, ok, ok, ok, ok, ok, 1024, ok, 1 << 20, None, 2, 16, 128, 64, 16,
                                 0, None) == 1
    assert lib.chord_b200_contiguous(odd, ok, ok, ok, ok, ok, 1024, ok, 1 << 20, None, 128, 128, 64, 2,
                                     0, None) == 1


def test_option_names_are_all_documented(native_lib):
    """Every option chord_b200_set_option accepts is listed in the header's comment."""
    header = (ROOT / "include" / "chord_b200.h").read_text()
    source = (ROOT / "chord_b200" / "csrc" / "core.cu").read_text()
    names = re.findall(r'std::strcmp\(name, "(\w+)"\)', source)
    assert len(names) >= 12
    for name in names:
        assert f'"{name}"' in header, f"option {name} is missing from include/chord_b200.h"
