"""The CPU oracle against the golden vectors produced by the reference's own code
(tests/golden/make_golden.py) and against itself (literal vs closed-form packer)."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import w4a16_oracle as O

GOLDEN = Path(__file__).resolve().parent / "golden"


def _bf16(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.copy()).view(torch.bfloat16)


def _f32(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.copy()).view(torch.float32)


def _load(name):
    z = np.load(GOLDEN / f"{name}.npz")
    e, n, k, m, top_k, block_m = (int(v) for v in z["shape"])
    codes = torch.from_numpy(O.unpack_checkpoint_uint4(z["checkpoint"])).reshape(e, n, k)
    return z, (e, n, k, m, top_k, block_m), codes


@pytest.mark.parametrize("name", ["tiny", "mid"])
def test_checkpoint_nibble_order_matches_reference(name):
    z, (e, n, k, *_), codes = _load(name)
    assert codes.min() >= 0 and codes.max() <= 15
    assert np.array_equal(O.pack_checkpoint_uint4(codes.numpy()), z["checkpoint"])


@pytest.mark.parametrize("name", ["tiny", "mid"])
def test_scale_permutation_matches_reference(name):
    z, _, _ = _load(name)
    got = O.permute_scale(_bf16(z["scale"]))
    assert torch.equal(got.view(torch.int16), torch.from_numpy(z["packed_scale"]))


@pytest.mark.parametrize("name", ["tiny", "mid"])
def test_routing_alignment_matches_reference(name):
    z, (e, n, k, m, top_k, block_m), _ = _load(name)
    topk = torch.from_numpy(z["topk_ids"])
    sorted_ids, expert_ids, padded = O.align_routing_blocks(topk, block_m, e)
    assert torch.equal(sorted_ids, torch.from_numpy(z["sorted_ids"]))
    assert torch.equal(expert_ids, torch.from_numpy(z["expert_ids"]))
    assert int(padded) == int(z["num_tokens_padded"])
    # the same draw comes out of the oracle's generator
    g = torch.Generator().manual_seed(m)
    assert torch.equal(O.topk_ids_random(m, top_k, e, g), topk)


@pytest.mark.parametrize("name", ["tiny", "mid"])
@pytest.mark.parametrize("projection", ["gate_up", "down"])
def test_indexed_reference_matches_reference(name, projection):
    z, (e, n, k, m, top_k, block_m), codes = _load(name)
    x = _bf16(z["x"] if projection == "gate_up" else z["x_routed"])
    scale = _bf16(z["scale"])
    topk = torch.from_numpy(z["topk_ids"])
    want = _f32(z["ref_" + projection])
    got = O.reference_indexed(x, codes, scale, topk, top_k, projection=projection)
    # Same products, FP32 sums in a different order (einsum vs matmul).
    assert O.max_abs_rel(got, want) < 1e-5
    rowwise = O.reference_indexed_rowwise(x, codes, scale, topk, top_k, projection=projection)
    assert O.max_abs_rel(rowwise, want) < 1e-6


@pytest.mark.parametrize("name", ["tiny", "mid"])
def test_fp32_dequant_matches_reference(name):
    z, (e, n, k, *_), codes = _load(name)
    got = O.dequant_reference_fp32(codes[0], _bf16(z["scale"])[0])
    assert torch.equal(got, _f32(z["dequant_fp32_e0"]))
    # and the BF16 dequantisation is its single rounding
    assert torch.equal(O.dequantize_bf16(codes[0], _bf16(z["scale"])[0]), got.to(torch.bfloat16))


def test_traffic_formula_matches_reference():
    z, (e, n, k, m, top_k, _), _ = _load("mid")
    assert O.traffic_bytes(e, n, k, m, m * top_k) == int(z["traffic"])
    assert O.cosine_diff(_f32(z["ref_gate_up"]), _f32(z["ref_gate_up"])) == float(z["cos_self"])


@pytest.mark.parametrize("shape", [(1, 64, 64), (2, 128, 128), (3, 192, 320)])
def test_closed_form_packer_equals_literal_kernel_emulation(shape):
    rng = np.random.default_rng(sum(shape))
    codes = rng.integers(0, 16, size=shape, dtype=np.int32)
    literal = O.repack_literal(codes)
    closed = O.repack_closed_form(codes)
    assert np.array_equal(literal, closed)
    assert np.array_equal(O.unpack_closed_form(closed, shape[1], shape[2]), codes)


def test_packed_word_layout_statement():
    """One word: rows r and r+8, K offsets {2q, 2q+1, 2q+8, 2q+9}; low half-word = even K."""
    codes = np.zeros((1, 64, 64), dtype=np.int32)
    n, k = 16 * 2 + 8 * 1 + 5, 16 * 3 + 8 * 1 + 2 * 2 + 1   # s=2, rh=1, r8=5 ; kb=3, kh=1, q=2, kk=1
    codes[0, n, k] = 0xF
    packed = O.repack_closed_form(codes).view(np.uint32)
    col = 4 * (4 * 5 + 2) + 2
    assert packed[0, 3, col] == 0xF << (4 * (2 * 1 + 1) + 16)
    assert np.count_nonzero(packed) == 1


def test_routing_contract_properties():
    g = torch.Generator().manual_seed(3)
    topk = O.topk_ids_random(200, 8, 384, g)
    for base, local in ((0, 48), (96, 48), (0, 384)):
        for block_m in (8, 16, 64):
            s, e, padded = O.align_routing_blocks(topk, block_m, local, base)
            assert int(padded) == s.numel() and s.numel() % block_m == 0
            valid = s[s < topk.numel()]
            assert valid.numel() == valid.unique().numel()
            want = ((topk.reshape(-1) >= base) & (topk.reshape(-1) < base + local)).sum()
            assert valid.numel() == int(want)
            blocks = s.view(-1, block_m) < topk.numel()
            assert not (blocks & ((~blocks).cumsum(1) > 0)).any()      # valid prefix, then sentinels
            assert blocks[:, 0].all()                                  # no empty block
            owners = topk.reshape(-1)[s.view(-1, block_m)[:, 0].long()] - base
            assert torch.equal(owners.to(torch.int32), e)


def test_empty_routing_is_allowed():
    topk = torch.full((4, 2), 300, dtype=torch.int32)
    s, e, padded = O.align_routing_blocks(topk, 16, 48, 0)
    assert s.numel() == 0 and e.numel() == 0 and int(padded) == 0
    with pytest.raises(ValueError):
        O.align_routing_blocks(topk, 16, 48, 0, allow_empty=False)


# ---- pinned by the reference's own GPU kernels (tests/golden/reference_gpu.npz, produced
# on a B200 by tests/golden/make_reference_gpu_golden.py from the reference's pack_w4a16
# and indexed)

def _reference_gpu():
    return np.load(Path(__file__).resolve().parent / "golden" / "reference_gpu.npz")


def _bf16(array):
    return torch.from_numpy(array.copy()).view(torch.bfloat16)


def test_packed_layout_equals_reference_gpu_packer():
    """Packed words and permuted scales, bit for bit, against the output of the
    reference's repack kernel (include/humming/kernel/repack.cuh) and
    _pack_weight_scale (operator/packing.py:45-52) run on a B200."""
    z = _reference_gpu()
    codes = O.unpack_checkpoint_uint4(torch.from_numpy(z["pack_words"]))
    codes = codes.numpy() if isinstance(codes, torch.Tensor) else codes
    assert np.array_equal(np.asarray(O.repack_closed_form(codes)), z["pack_packed"])
    assert np.array_equal(np.asarray(O.repack_literal(codes)), z["pack_packed"])
    scale_out = O.permute_scale(_bf16(z["pack_scale_in"]))
    assert np.array_equal(scale_out.contiguous().view(torch.int16).numpy(), z["pack_scale_out"])
    # and back: the closed-form inverse recovers the codes from the reference's words
    assert np.array_equal(np.asarray(O.unpack_closed_form(z["pack_packed"], 256, 320)), codes)


def test_oracle_indexed_matches_reference_gpu_kernel():
    """The CPU restatement against the BF16 output of the reference's own `indexed`
    kernel (its Blackwell mma.sync schedule) on a B200: same rows written, cosine
    difference <= 5e-3 (the reference's own limit, tests/test_w4a16_indexed.py:63)."""
    z = _reference_gpu()
    e, n, k, m, top_k, block_m = (int(v) for v in z["idx_shape"])
    codes = O.unpack_checkpoint_uint4(torch.from_numpy(z["idx_words"]))
    codes = codes if isinstance(codes, torch.Tensor) else torch.from_numpy(np.asarray(codes))
    topk = torch.from_numpy(z["idx_topk"].astype(np.int64))
    sorted_ids, expert_ids, padded = O.align_routing_blocks(topk, block_m, e, 0)
    assert np.array_equal(sorted_ids.numpy(), z["idx_sorted_ids"])
    assert np.array_equal(expert_ids.numpy(), z["idx_expert_ids"])
    assert int(padded) == int(z["idx_num_tokens_padded"][0])
    ref = O.reference_indexed(_bf16(z["idx_x"]), codes, _bf16(z["idx_scale"]), topk, top_k)
    got = _bf16(z["idx_out"]).float()
    assert got.shape == ref.shape == (m * top_k, n)
    assert O.cosine_diff(got, ref) <= 5e-3
    assert O.max_abs_rel(got, ref) <= 1e-2


# ------------------------------------------------- masked / contiguous goldens --

from tests.cases import load_grouped_golden  # noqa: E402


@pytest.mark.parametrize("name", ["masked_a", "masked_b"])
def test_masked_reference_matches_the_references_own_test_vectors(name):
    """`reference_masked` against tests/test_w4a16_grouped.py::make_masked_case run on the
    CPU: the same rows are written (the reference leaves the others zero), the FP32-dequant
    form reproduces its BF16 values to one rounding, and the BF16-dequant form the kernels
    implement stays inside the reference's own limit (cos-diff < 1e-3)."""
    c = load_grouped_golden(name)
    ref = c["ref"].float()
    loose = O.reference_masked(c["x"], c["codes"], c["scale"], c["masked_m"], dequant="fp32")
    exact = O.reference_masked(c["x"], c["codes"], c["scale"], c["masked_m"])
    written = ~torch.isnan(exact).any(dim=2)
    for g in range(c["groups"]):
        mm = int(c["masked_m"][g])
        assert bool(written[g, :mm].all()) and not bool(written[g, mm:].any())
        assert bool((ref[g, mm:] == 0).all())
    assert torch.equal(torch.isnan(loose), torch.isnan(exact))
    got = loose[written].to(torch.bfloat16).float()
    # same products, different summation order: at most one BF16 step apart
    assert bool(((got - ref[written]).abs() <= ref[written].abs() * 2 ** -7 + 1e-6).all())
    assert O.cosine_diff(exact[written], ref[written]) < c["cosine_limit"]
    assert O.max_abs_rel(exact[written], ref[written]) <= 1e-2


@pytest.mark.parametrize("name", ["contiguous_a", "contiguous_b"])
def test_contiguous_reference_matches_the_references_own_test_vectors(name):
    """`reference_contiguous` against make_contiguous_case: every 128-row tile of an expert
    is written, its rows up to the expert's count carry x . W^T, its padding rows (index
    -1, zeroed activations) come out as zeros - what the reference expects there."""
    c = load_grouped_golden(name)
    ref = c["ref"].float()
    loose = O.reference_contiguous(c["x"], c["codes"], c["scale"], c["m_indices"], dequant="fp32")
    exact = O.reference_contiguous(c["x"], c["codes"], c["scale"], c["m_indices"])
    assert not bool(torch.isnan(exact).any())  # every tile of these cases starts with a valid row
    pad = c["m_indices"] < 0
    assert bool((exact[pad] == 0).all()) and bool((ref[pad] == 0).all())
    for expert, start, end in c["bounds"]:
        assert bool((c["m_indices"][start:end] == expert).all())
    got = loose.to(torch.bfloat16).float()
    assert bool(((got - ref).abs() <= ref.abs() * 2 ** -7 + 1e-6).all())
    assert O.cosine_diff(exact[~pad], ref[~pad]) < c["cosine_limit"]
    assert O.max_abs_rel(exact[~pad], ref[~pad]) <= 1e-2
