"""``pack_w4a16`` and ``PreparedWeight``: same interface as
chord_kernels/operator/packing.py:26-138, on the sm_100a packer kernels."""

from __future__ import annotations

import dataclasses
from collections.abc import Iterator

import torch

from . import _checks, _lib


@dataclasses.dataclass(frozen=True, eq=False)
class PreparedWeight:
    """Packed weight ``[E, K/16, 2N]`` and scale ``[E, K/32, N]``; every operator
    (indexed, contiguous, masked) reads the same bytes (packing.py:26-42)."""

    packed: torch.Tensor
    scale: torch.Tensor
    n: int
    k: int
    num_experts: int

    @property
    def tensors(self) -> tuple[torch.Tensor, torch.Tensor]:
        return self.packed, self.scale

    def __iter__(self) -> Iterator[torch.Tensor]:
        return iter(self.tensors)


def pack_w4a16(
    weight_uint4: torch.Tensor,
    weight_scale: torch.Tensor,
    *,
    packed: bool = False,
) -> PreparedWeight:
    """Pack INT4 weights and their BF16 group-32 scales.

    ``weight_uint4`` is int32 ``[E, N, K]`` holding unsigned codes in ``[0, 15]``
    (decoded as ``code - 8``), or with ``packed=True`` the checkpoint form
    ``[E, N, K/8]``, eight little-endian nibbles per word.  ``weight_scale`` is
    BF16 ``[E, N, K/32]``.  Argument checks and exception classes follow
    packing.py:68-117.
    """
    _checks.flag("packed", packed)
    layout = "[E, N, K/8]" if packed else "[E, N, K]"
    weight_uint4 = _checks.tensor("weight_uint4", weight_uint4, dtype=torch.int32, cuda=False,
                                  contiguous=False)
    _checks.tensor("weight_scale", weight_scale, cuda=False, contiguous=False)
    if weight_uint4.ndim != 3:
        raise ValueError(f"weight_uint4 must have shape {layout}, got {tuple(weight_uint4.shape)}")
    if not weight_uint4.is_cuda or not weight_uint4.is_contiguous():
        raise ValueError("weight_uint4 must be a contiguous CUDA tensor")
    _checks.supported_gpu(weight_uint4.device)
    num_experts, shape_n, stored_k = weight_uint4.shape
    if 0 in (num_experts, shape_n, stored_k):
        raise ValueError(f"weight_uint4 dimensions must be non-zero, got {tuple(weight_uint4.shape)}")
    shape_k = stored_k * (8 if packed else 1)
    for name, extent, unit in (("shape_n", shape_n, 128), ("shape_k", shape_k, 64)):
        if extent % unit:
            raise ValueError(f"{name} must be divisible by {unit}, got {extent}")
    scale_shape = (num_experts, shape_n, shape_k // 32)
    if tuple(weight_scale.shape) != scale_shape:
        raise ValueError(f"weight_scale must have shape {scale_shape}, got {tuple(weight_scale.shape)}")
    _checks.tensor("weight_scale", weight_scale, dtype=torch.bfloat16, device=weight_uint4.device)

    lib = _lib.load()
    device = weight_uint4.device
    packed_weight = torch.empty(
        (num_experts, shape_k // 16, shape_n * 2), dtype=torch.int32, device=device
    )
    packed_scale = torch.empty(
        (num_experts, shape_k // 32, shape_n), dtype=torch.bfloat16, device=device
    )
    with torch.cuda.device(device):
        stream = _lib.stream_handle(device)
        # The range check the reference does with torch.aminmax (packing.py:111-117)
        # rides along in the packer; only its verdict is read back.
        range_flag = None if packed else torch.zeros(1, dtype=torch.int32, device=device)
        _lib.check(lib.chord_b200_repack_w4a16(
            weight_uint4.data_ptr(), packed_weight.data_ptr(), num_experts, shape_n, shape_k,
            1 if packed else 0, 0 if range_flag is None else range_flag.data_ptr(), stream,
        ))
        _lib.check(lib.chord_b200_permute_scale(
            weight_scale.data_ptr(), packed_scale.data_ptr(), num_experts, shape_n, shape_k, stream,
        ))
        if range_flag is not None and int(range_flag.item()) != 0:
            minimum, maximum = torch.aminmax(weight_uint4)
            raise ValueError(
                "weight_uint4 values must be in [0, 15], got "
                f"[{minimum.item()}, {maximum.item()}]"
            )
    return PreparedWeight(
        packed=packed_weight, scale=packed_scale, n=shape_n, k=shape_k, num_experts=num_experts
    )


__all__ = ["PreparedWeight", "pack_w4a16"]
