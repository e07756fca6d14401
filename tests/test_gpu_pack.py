"""Packer parity on the GPU: packed bytes bit-exact against the oracle for both input
forms (the reference's own check is that both forms give identical bytes,
tests/test_w4a16_indexed.py:369-372), scales bit-exact, range check, round trip."""

import numpy as np
import pytest
import torch

from oracle import w4a16_oracle as O
from tests.cases import make_checkpoint_weights, make_weights

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(1, 128, 64), (2, 128, 128), (3, 256, 320), (2, 1024, 512),
                                   (8, 1024, 512), (5, 384, 2368)])
def test_packed_bytes_bit_exact_both_input_forms(device, shape):
    import chord_b200

    e, n, k = shape
    codes, scale = make_weights(e, n, k, seed=e * 1000 + n + k)
    want = torch.from_numpy(O.repack_closed_form(codes.numpy()))
    unpacked = chord_b200.pack_w4a16(codes.to(device), scale.to(device))
    checkpoint = torch.from_numpy(O.pack_checkpoint_uint4(codes.numpy()))
    packed = chord_b200.pack_w4a16(checkpoint.to(device), scale.to(device), packed=True)
    assert unpacked.packed.shape == (e, k // 16, 2 * n) and unpacked.packed.dtype == torch.int32
    assert torch.equal(unpacked.packed.cpu(), want)
    assert torch.equal(packed.packed, unpacked.packed)
    assert torch.equal(unpacked.scale.cpu().view(torch.int16),
                       O.permute_scale(scale).view(torch.int16))
    assert (unpacked.n, unpacked.k, unpacked.num_experts) == (n, k, e)


def test_full_size_expert_round_trip(device):
    """K2.5 gate_up shape, four experts, checkpoint form: unpacking the packed words
    gives back every nibble (size-independent property; no full CPU repack needed)."""
    import chord_b200

    e, n, k = 4, 4096, 7168
    words, scale = make_checkpoint_weights(e, n, k, seed=11)
    w = chord_b200.pack_w4a16(words.to(device), scale.to(device), packed=True)
    codes = O.unpack_closed_form(w.packed.cpu().numpy(), n, k)
    assert np.array_equal(O.pack_checkpoint_uint4(codes), words.numpy())


def test_range_check_and_argument_errors(device):
    import chord_b200

    scale = torch.ones((1, 128, 2), dtype=torch.bfloat16, device=device)
    with pytest.raises(ValueError, match=r"\[0, 15\]"):
        chord_b200.pack_w4a16(torch.full((1, 128, 64), 16, dtype=torch.int32, device=device), scale)
    with pytest.raises(ValueError, match=r"\[0, 15\]"):
        chord_b200.pack_w4a16(torch.full((1, 128, 64), -1, dtype=torch.int32, device=device), scale)
    ok = torch.zeros((1, 128, 64), dtype=torch.int32, device=device)
    with pytest.raises(ValueError, match="divisible by 128"):
        chord_b200.pack_w4a16(ok[:, :64].contiguous(), scale[:, :64].contiguous())
    with pytest.raises(ValueError, match="divisible by 64"):
        chord_b200.pack_w4a16(ok[:, :, :32].contiguous(), scale[:, :, :1].contiguous())
    with pytest.raises(ValueError, match="weight_scale must have shape"):
        chord_b200.pack_w4a16(ok, scale[:, :, :1].contiguous())
    with pytest.raises(TypeError):
        chord_b200.pack_w4a16(ok, scale.float())


def test_packer_equals_reference_gpu_packer(device):
    """Bit-exact against the packed words and scales the reference's own pack_w4a16
    produced on a B200 (tests/golden/reference_gpu.npz)."""
    from pathlib import Path

    import chord_b200

    z = np.load(Path(__file__).resolve().parent / "golden" / "reference_gpu.npz")
    scale = torch.from_numpy(z["pack_scale_in"].copy()).view(torch.bfloat16)
    words = torch.from_numpy(z["pack_words"])
    got = chord_b200.pack_w4a16(words.to(device), scale.to(device), packed=True)
    assert np.array_equal(got.packed.cpu().numpy(), z["pack_packed"])
    assert np.array_equal(got.scale.cpu().contiguous().view(torch.int16).numpy(), z["pack_scale_out"])
    codes = O.unpack_checkpoint_uint4(words)
    codes = codes if isinstance(codes, torch.Tensor) else torch.from_numpy(np.asarray(codes))
    got2 = chord_b200.pack_w4a16(codes.to(torch.int32).to(device), scale.to(device))
    assert np.array_equal(got2.packed.cpu().numpy(), z["pack_packed"])


def test_indexed_agrees_with_reference_gpu_kernel(device):
    """Same inputs and routing as the reference's own `indexed` launch on a B200: the
    same rows are written, outputs agree within the BF16 output rounding (both round an
    FP32 sum once; the summation orders differ)."""
    from pathlib import Path

    import chord_b200

    z = np.load(Path(__file__).resolve().parent / "golden" / "reference_gpu.npz")
    e, n, k, m, top_k, block_m = (int(v) for v in z["idx_shape"])
    bf = lambda a: torch.from_numpy(a.copy()).view(torch.bfloat16)  # noqa: E731
    weight = chord_b200.pack_w4a16(torch.from_numpy(z["idx_words"]).to(device), bf(z["idx_scale"]).to(device),
                                   packed=True)
    out = torch.full((m * top_k, n), float("nan"), dtype=torch.bfloat16, device=device)
    chord_b200.indexed(bf(z["idx_x"]).to(device), weight, torch.from_numpy(z["idx_sorted_ids"]).to(device),
                       torch.from_numpy(z["idx_expert_ids"]).to(device),
                       torch.from_numpy(z["idx_num_tokens_padded"]).to(device), top_k, outputs=out,
                       block_m=block_m)
    torch.cuda.synchronize()
    got, ref = out.float().cpu(), bf(z["idx_out"]).float()
    assert not torch.isnan(got).any()
    assert O.cosine_diff(got, ref) <= 1e-5
    assert O.max_abs_rel(got, ref) <= 1e-2
