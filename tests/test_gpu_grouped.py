"""`masked` and `contiguous` on the GPU against the CPU oracle, plus the point of
packing once: one PreparedWeight serves all three operators
(reference: tests/test_w4a16_grouped.py:407-623; its limit is cos-diff < 1e-3)."""

import pytest
import torch

from oracle import w4a16_oracle as O
from tests.cases import (load_grouped_golden, make_contiguous_case, make_indexed_case,
                         make_masked_case)

pytestmark = pytest.mark.gpu

COS_LIMIT = 1e-3
REL_LIMIT = 1e-2


def _status_ok(device):
    from chord_b200.indexed_gemm import status_word

    torch.cuda.synchronize()
    assert int(status_word(device).item()) == 0


def _compare(got, ref):
    got = got.float().cpu()
    written = ~torch.isnan(got).any(dim=1)
    expected = ~torch.isnan(ref).any(dim=1)
    assert torch.equal(written, expected)
    if expected.any():
        assert O.cosine_diff(got[expected], ref[expected]) < COS_LIMIT
        assert O.max_abs_rel(got[expected], ref[expected]) <= REL_LIMIT


@pytest.mark.parametrize("groups,max_m,n,k,expected_m", [
    (6, 40, 512, 256, 8), (12, 256, 1024, 512, 32), (4, 256, 512, 1024, 128),
    (3, 8, 256, 128, 8), (5, 24, 256, 192, 16), (2, 300, 256, 256, 300),
])
def test_masked_matches_oracle(device, groups, max_m, n, k, expected_m):
    import chord_b200

    case = make_masked_case(groups, max_m, n, k, expected_m, seed=groups * 7 + max_m)
    w = chord_b200.pack_w4a16(case["codes"].to(device), case["scale"].to(device))
    out = torch.full((groups * max_m, n), float("nan"), dtype=torch.bfloat16, device=device)
    res = chord_b200.masked(case["x3"].to(device), w, case["masked_m"].to(device), expected_m,
                            outputs=out)
    _status_ok(device)
    assert res.shape == (groups * max_m, n) and res.data_ptr() == out.data_ptr()
    ref = O.reference_masked(case["x3"], case["codes"], case["scale"], case["masked_m"])
    _compare(out, ref.reshape(groups * max_m, n))


def test_masked_ragged_groups_flat_input_and_repeatability(device):
    """Ragged counts including empty and full groups, flat [G*max_m, K] input, int64
    masked_m (cast like the reference does), three launches bit-equal."""
    import chord_b200

    groups, max_m, n, k = 48, 40, 256, 256
    case = make_masked_case(groups, max_m, n, k, 8, seed=5)
    case["masked_m"] = torch.tensor([(i * 7) % 41 for i in range(groups)], dtype=torch.int32)
    w = chord_b200.pack_w4a16(case["codes"].to(device), case["scale"].to(device))
    flat = case["x3"].reshape(groups * max_m, k).to(device)
    outs = []
    for _ in range(3):
        out = torch.full((groups * max_m, n), float("nan"), dtype=torch.bfloat16, device=device)
        chord_b200.masked(flat, w, case["masked_m"].long().to(device), 8, outputs=out)
        outs.append(out)
    _status_ok(device)
    ref = O.reference_masked(case["x3"], case["codes"], case["scale"], case["masked_m"])
    _compare(outs[0], ref.reshape(groups * max_m, n))
    for other in outs[1:]:
        assert torch.equal(other.view(torch.int16), outs[0].view(torch.int16))


@pytest.mark.parametrize("counts,n,k,extra", [
    ([128, 7, 300, 0, 129], 512, 512, 1), ([128] * 6, 256, 1024, 0), ([1], 128, 64, 0),
    ([256, 512], 384, 2368, 0),
])
def test_contiguous_matches_oracle(device, counts, n, k, extra):
    import chord_b200

    case = make_contiguous_case(counts, n, k, seed=len(counts) + n, extra_padding_tiles=extra)
    w = chord_b200.pack_w4a16(case["codes"].to(device), case["scale"].to(device))
    m = case["x2"].size(0)
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=device)
    chord_b200.contiguous(case["x2"].to(device), w, case["m_indices"].to(device), outputs=out)
    _status_ok(device)
    ref = O.reference_contiguous(case["x2"], case["codes"], case["scale"], case["m_indices"])
    _compare(out, ref)
    # padding rows of a live tile come out as exact zeros (their inputs are zero)
    got = out.float().cpu()
    pad = (case["m_indices"] < 0) & ~torch.isnan(got).any(dim=1)
    assert bool((got[pad] == 0).all())


def test_one_packed_weight_serves_all_three_operators(device):
    import chord_b200

    e, n, k = 4, 256, 512
    icase = make_indexed_case(num_experts=e, n=n, k=k, m=32, top_k=2, block_m=16, seed=40)
    w = chord_b200.pack_w4a16(icase["codes"].to(device), icase["scale"].to(device))
    locks = torch.zeros(1024, dtype=torch.int32, device=device)
    out = torch.full((64, n), float("nan"), dtype=torch.bfloat16, device=device)
    chord_b200.indexed(icase["x"].to(device), w, icase["sorted_ids"].to(device),
                       icase["expert_ids"].to(device), icase["num_tokens_padded"].to(device).reshape(1),
                       2, locks=locks, outputs=out, block_m=16)
    ref = O.reference_indexed(icase["x"], icase["codes"], icase["scale"], icase["topk_ids"], 2)
    _compare(out, ref)

    g = torch.Generator().manual_seed(41)
    x3 = torch.randn((e, 16, k), generator=g).to(torch.bfloat16)
    mm = torch.tensor([16, 3, 0, 9], dtype=torch.int32)
    out = torch.full((e * 16, n), float("nan"), dtype=torch.bfloat16, device=device)
    chord_b200.masked(x3.to(device), w, mm.to(device), 8, outputs=out)
    _compare(out, O.reference_masked(x3, icase["codes"], icase["scale"], mm).reshape(e * 16, n))

    x2 = torch.randn((e * 128, k), generator=g).to(torch.bfloat16)
    mi = torch.arange(e, dtype=torch.int32).repeat_interleave(128)
    got = chord_b200.contiguous(x2.to(device), w, mi.to(device))
    _compare(got, O.reference_contiguous(x2, icase["codes"], icase["scale"], mi))
    _status_ok(device)


def test_grouped_argument_checks(device):
    import chord_b200

    case = make_masked_case(2, 8, 128, 64, 8, seed=1)
    w = chord_b200.pack_w4a16(case["codes"].to(device), case["scale"].to(device))
    x3 = case["x3"].to(device)
    mm = case["masked_m"].to(device)
    with pytest.raises(ValueError, match="expected_m"):
        chord_b200.masked(x3, w, mm, 0)
    with pytest.raises(TypeError):
        chord_b200.masked(x3, w, mm, 8.0)
    with pytest.raises(ValueError, match="groups"):
        chord_b200.masked(x3[:1].contiguous(), w, mm, 8)
    with pytest.raises(ValueError, match="masked_m"):
        chord_b200.masked(x3, w, mm[:1].contiguous(), 8)
    with pytest.raises(ValueError, match="128-aligned"):
        chord_b200.contiguous(x3.reshape(16, 64), w, torch.zeros(16, dtype=torch.int32, device=device))
    with pytest.raises(ValueError, match="m_indices"):
        chord_b200.contiguous(torch.zeros((128, 64), dtype=torch.bfloat16, device=device), w,
                              torch.zeros(64, dtype=torch.int32, device=device))


@pytest.mark.parametrize("option,value", [("ksplit", 0), ("contiguous_tile", 256), ("npair", 0), ("decode_kernel", 0),
                                          ("pair", 0)])
def test_grouped_kernel_variants(device, option, value):
    """Without the second MMA issuer / with merged 256-token tiles (on CTA pairs) for every
    expert / with one weight block per tile / with small masked tiles on the general kernel /
    without CTA pairs (256-token tiles on one CTA, `contiguous` in one launch): same results
    within tolerance."""
    import chord_b200
    from chord_b200 import _lib

    defaults = {"ksplit": 1, "contiguous_tile": 0, "npair": 1, "decode_kernel": 1, "pair": 1}
    ccase = make_contiguous_case([5, 300, 0, 128, 77, 513], 512, 640, seed=31)
    mcase = make_masked_case(6, 200, 256, 384, 16, seed=32)
    mcase["masked_m"] = torch.tensor([0, 3, 16, 33, 150, 200], dtype=torch.int32)
    _lib.set_option(option, value)
    try:
        w = chord_b200.pack_w4a16(ccase["codes"].to(device), ccase["scale"].to(device))
        out = torch.full((ccase["x2"].size(0), 512), float("nan"), dtype=torch.bfloat16, device=device)
        chord_b200.contiguous(ccase["x2"].to(device), w, ccase["m_indices"].to(device), outputs=out)
        _status_ok(device)
        _compare(out, O.reference_contiguous(ccase["x2"], ccase["codes"], ccase["scale"], ccase["m_indices"]))
        for expected_m in (16, 200):
            wm = chord_b200.pack_w4a16(mcase["codes"].to(device), mcase["scale"].to(device))
            mout = torch.full((6 * 200, 256), float("nan"), dtype=torch.bfloat16, device=device)
            chord_b200.masked(mcase["x3"].to(device), wm, mcase["masked_m"].to(device), expected_m,
                              outputs=mout)
            _status_ok(device)
            ref = O.reference_masked(mcase["x3"], mcase["codes"], mcase["scale"], mcase["masked_m"])
            _compare(mout, ref.reshape(6 * 200, 256))
    finally:
        _lib.set_option(option, defaults[option])


@pytest.mark.parametrize("name", ["masked_a", "masked_b"])
def test_masked_matches_the_references_own_test_vectors(device, name):
    """Inputs and expected outputs built by the reference's make_masked_case on the CPU
    (tests/golden/grouped.npz): rows below masked_m within its limit (cos-diff < 1e-3
    against its FP32-dequantised expectation), rows at or above masked_m untouched."""
    import chord_b200

    c = load_grouped_golden(name)
    w = chord_b200.pack_w4a16(c["codes"].to(device), c["scale"].to(device))
    out = torch.full((c["groups"] * c["max_m"], c["n"]), float("nan"), dtype=torch.bfloat16, device=device)
    chord_b200.masked(c["x"].to(device), w, c["masked_m"].to(device), c["expected_m"], outputs=out)
    _status_ok(device)
    got = out.float().cpu().view(c["groups"], c["max_m"], c["n"])
    ref = c["ref"].float()
    for g in range(c["groups"]):
        mm = int(c["masked_m"][g])
        assert not bool(torch.isnan(got[g, :mm]).any())
        assert bool(torch.isnan(got[g, mm:]).all())
        assert O.cosine_diff(got[g, :mm], ref[g, :mm]) < c["cosine_limit"]
        assert O.max_abs_rel(got[g, :mm], ref[g, :mm]) <= REL_LIMIT


@pytest.mark.parametrize("name", ["contiguous_a", "contiguous_b"])
def test_contiguous_matches_the_references_own_test_vectors(device, name):
    """Same for make_contiguous_case: every row of the output equals the reference's
    expectation, which is zero on the padding rows (index -1) of an expert's run."""
    import chord_b200

    c = load_grouped_golden(name)
    w = chord_b200.pack_w4a16(c["codes"].to(device), c["scale"].to(device))
    m = c["x"].size(0)
    out = torch.full((m, c["n"]), float("nan"), dtype=torch.bfloat16, device=device)
    chord_b200.contiguous(c["x"].to(device), w, c["m_indices"].to(device), outputs=out)
    _status_ok(device)
    got, ref = out.float().cpu(), c["ref"].float()
    assert not bool(torch.isnan(got).any())
    pad = c["m_indices"] < 0
    assert bool((got[pad] == ref[pad]).all())
    assert O.cosine_diff(got[~pad], ref[~pad]) < c["cosine_limit"]
    assert O.max_abs_rel(got[~pad], ref[~pad]) <= REL_LIMIT


def test_cta_pairs_agree_with_single_ctas(device):
    """K >= 2048, where tiles of more than 128 tokens run as clusters of two CTAs
    (tcgen05.mma.cta_group::2, half of the token rows loaded by each CTA, two groups of
    epilogue warps): `contiguous` with experts of several 128-row blocks (a launch of their
    own; single-block experts keep the 128-token layout) and `masked` with 256-token tiles.
    Against the same calls without CTA pairs: the same rows written, values equal up to the
    order of the stream-K partial sums; against the oracle; status word clear and locks back
    at zero, twice in a row."""
    import chord_b200
    from chord_b200 import _lib
    from chord_b200.indexed_gemm import default_locks

    case = make_contiguous_case([256, 40, 700, 0, 128, 129, 1], 1024, 2368, seed=77)  # last K stage half-filled
    mcase = make_masked_case(5, 256, 512, 2048, 200, seed=78)
    mcase["masked_m"] = torch.tensor([256, 0, 131, 200, 7], dtype=torch.int32)
    w = chord_b200.pack_w4a16(case["codes"].to(device), case["scale"].to(device))
    wm = chord_b200.pack_w4a16(mcase["codes"].to(device), mcase["scale"].to(device))
    x2, m_indices = case["x2"].to(device), case["m_indices"].to(device)
    x3, masked_m = mcase["x3"].to(device), mcase["masked_m"].to(device)
    outs, mouts = {}, {}
    try:
        for pair in (0, 1):
            _lib.set_option("pair", pair)
            for _ in range(2):
                out = torch.full((x2.size(0), 1024), float("nan"), dtype=torch.bfloat16, device=device)
                chord_b200.contiguous(x2, w, m_indices, outputs=out)
                _status_ok(device)
                mout = torch.full((5 * 256, 512), float("nan"), dtype=torch.bfloat16, device=device)
                chord_b200.masked(x3, wm, masked_m, 200, outputs=mout)
                _status_ok(device)
            assert bool((default_locks(device) == 0).all())
            outs[pair], mouts[pair] = out.float().cpu(), mout.float().cpu()
    finally:
        _lib.set_option("pair", 1)
    for got in (outs, mouts):
        assert torch.equal(torch.isnan(got[0]), torch.isnan(got[1]))
        a, b = got[0].nan_to_num(), got[1].nan_to_num()
        assert float((a == b).float().mean()) >= 0.995
        assert float((a - b).abs().max()) <= 2.0 ** -6 * float(a.abs().max())
    _compare(outs[1].to(torch.bfloat16),
             O.reference_contiguous(case["x2"], case["codes"], case["scale"], case["m_indices"]))
    ref = O.reference_masked(mcase["x3"], mcase["codes"], mcase["scale"], mcase["masked_m"])
    _compare(mouts[1].to(torch.bfloat16), ref.reshape(5 * 256, 512))


def test_programmatic_dependent_launch_does_not_change_grouped_results(device):
    """`enable_pdl=True` on `contiguous` (two launches, the second on clusters of two CTAs)
    and `masked` (256-token tiles on clusters): the launch attribute only lets a kernel's
    set-up overlap its predecessor's tail, so the outputs are bit-equal to plain launches."""
    import chord_b200

    case = make_contiguous_case([256, 40, 700, 0, 128, 129, 1], 1024, 2368, seed=77)
    mcase = make_masked_case(5, 256, 512, 2048, 200, seed=78)
    w = chord_b200.pack_w4a16(case["codes"].to(device), case["scale"].to(device))
    wm = chord_b200.pack_w4a16(mcase["codes"].to(device), mcase["scale"].to(device))
    x2, m_indices = case["x2"].to(device), case["m_indices"].to(device)
    x3, masked_m = mcase["x3"].to(device), mcase["masked_m"].to(device)
    results = {}
    for pdl in (False, True):
        for _ in range(3):          # back to back, so that a launch does follow a running kernel
            out = torch.full((x2.size(0), 1024), float("nan"), dtype=torch.bfloat16, device=device)
            chord_b200.contiguous(x2, w, m_indices, outputs=out, enable_pdl=pdl)
            mout = torch.full((5 * 256, 512), float("nan"), dtype=torch.bfloat16, device=device)
            chord_b200.masked(x3, wm, masked_m, 200, outputs=mout, enable_pdl=pdl)
        _status_ok(device)
        results[pdl] = (out, mout)
    for plain, overlapped in zip(results[False], results[True]):
        assert torch.equal(plain.view(torch.int16), overlapped.view(torch.int16))
