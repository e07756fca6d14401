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
