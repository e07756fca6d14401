"""``masked`` / ``contiguous`` grouped W4A16 GEMMs, same interface as
chord_kernels/ops.py:49-90 and chord_kernels/operator/grouped/api.py:116-271.

The reference implements these for SM90 only (WGMMA); here they run on the same
sm_100a tcgen05 kernel as ``indexed`` with a different tile scheduler."""

from __future__ import annotations

import torch

from . import _lib
from .indexed_gemm import gemm_scratch, status_word
from .packing import PreparedWeight, _validate_supported_architecture


def _check_weight(weight: PreparedWeight, device: torch.device) -> None:
    """Shape/dtype checks of chord_kernels/operator/grouped/api.py:24-60 (the SM90
    gate and its BLOCK_K rule do not apply: K % 64 is all this kernel needs)."""
    if not isinstance(weight, PreparedWeight):
        raise TypeError("weight must be a PreparedWeight from pack_w4a16()")
    _validate_supported_architecture(device)
    packed, scale = weight.packed, weight.scale
    if packed.dtype != torch.int32 or scale.dtype != torch.bfloat16:
        raise TypeError(
            f"packed weight must be int32 and scale bfloat16, got {packed.dtype}/{scale.dtype}"
        )
    if (tuple(packed.shape) != (weight.num_experts, weight.k // 16, weight.n * 2)
            or tuple(scale.shape) != (weight.num_experts, weight.k // 32, weight.n)):
        raise ValueError(
            "packed tensors disagree with the recorded metadata: "
            f"packed {tuple(packed.shape)} vs {(weight.num_experts, weight.k // 16, weight.n * 2)}, "
            f"scale {tuple(scale.shape)} vs {(weight.num_experts, weight.k // 32, weight.n)}"
        )
    for name, tensor in (("packed weight", packed), ("scale", scale)):
        if tensor.device != device or not tensor.is_contiguous():
            raise ValueError(f"{name} must be contiguous and on {device}")


def _check_activation(inputs: torch.Tensor, shape_k: int) -> None:
    if not isinstance(inputs, torch.Tensor):
        raise TypeError(f"inputs must be a torch.Tensor, got {type(inputs).__name__}")
    if inputs.dtype != torch.bfloat16:
        raise TypeError(f"inputs must be bfloat16, got {inputs.dtype}")
    if not inputs.is_cuda or not inputs.is_contiguous():
        raise ValueError("inputs must be a contiguous CUDA tensor")
    if inputs.size(-1) != shape_k:
        raise ValueError(f"inputs K={inputs.size(-1)} != weight K={shape_k}")
    if inputs.size(-1) == 0 or inputs.numel() == 0:
        raise ValueError("inputs must be non-empty")


def _check_outputs(outputs, shape, device):
    if not isinstance(outputs, torch.Tensor) or outputs.dtype != torch.bfloat16:
        raise TypeError("outputs must be a torch.bfloat16 tensor")
    if outputs.device != device or not outputs.is_contiguous() or outputs.numel() != shape[0] * shape[1]:
        raise ValueError(f"outputs must be contiguous BF16 with {shape[0] * shape[1]} elements on {device}")


def masked_tile_m(expected_m: int) -> int:
    return int(_lib.load().chord_b200_masked_tile_m(expected_m))


def w4a16_masked(
    inputs: torch.Tensor,
    weight: PreparedWeight,
    masked_m: torch.Tensor,
    expected_m: int,
    *,
    outputs: torch.Tensor | None = None,
    enable_pdl: bool = False,
) -> torch.Tensor:
    """Masked (decode) grouped GEMM: ``[G*max_m, K]`` or ``[G, max_m, K]`` in, flat
    ``[G*max_m, N]`` out.  ``masked_m`` ``[G] int32`` is each group's valid rows;
    ``expected_m`` only sizes the tiles.  Rows past ``masked_m[g]`` are not written.
    """
    if not isinstance(inputs, torch.Tensor):
        raise TypeError(f"inputs must be a torch.Tensor, got {type(inputs).__name__}")
    _check_weight(weight, inputs.device)
    _check_activation(inputs, weight.k)
    if inputs.dim() == 2:
        if inputs.size(0) % weight.num_experts:
            raise ValueError(
                f"flat inputs rows {inputs.size(0)} are not divisible by "
                f"num_experts={weight.num_experts}"
            )
        grouped = inputs.view(weight.num_experts, inputs.size(0) // weight.num_experts, weight.k)
    elif inputs.dim() == 3:
        if inputs.size(0) != weight.num_experts:
            raise ValueError(f"inputs groups {inputs.size(0)} != num_experts={weight.num_experts}")
        grouped = inputs
    else:
        raise ValueError(f"inputs must be 2D or 3D, got {inputs.dim()}D")
    if not isinstance(masked_m, torch.Tensor):
        raise TypeError(f"masked_m must be a torch.Tensor, got {type(masked_m).__name__}")
    if masked_m.dtype != torch.int32:
        masked_m = masked_m.to(torch.int32)
    if (masked_m.dim() != 1 or masked_m.numel() != weight.num_experts or not masked_m.is_cuda
            or not masked_m.is_contiguous()):
        raise ValueError(f"masked_m must be contiguous CUDA int32 [{weight.num_experts}]")
    if isinstance(expected_m, bool) or not isinstance(expected_m, int):
        raise TypeError(f"expected_m must be an int, got {type(expected_m).__name__}")
    if expected_m <= 0:
        raise ValueError(f"expected_m must be positive, got {expected_m}")
    if not isinstance(enable_pdl, bool):
        raise TypeError(f"enable_pdl must be a bool, got {type(enable_pdl).__name__}")

    device = inputs.device
    groups, max_m = grouped.size(0), grouped.size(1)
    if outputs is None:
        outputs = torch.empty((groups * max_m, weight.n), dtype=torch.bfloat16, device=device)
    else:
        _check_outputs(outputs, (groups * max_m, weight.n), device)
    tile_m = masked_tile_m(expected_m)
    lib = _lib.load()
    with torch.cuda.device(device):
        locks, workspace, ws_bytes = gemm_scratch(device, tile_m, None)
        _lib.check(lib.chord_b200_masked(
            grouped.data_ptr(), weight.packed.data_ptr(), weight.scale.data_ptr(),
            masked_m.data_ptr(), outputs.data_ptr(), locks.data_ptr(), locks.numel(),
            workspace.data_ptr(), ws_bytes, status_word(device).data_ptr(),
            groups, max_m, weight.n, weight.k, tile_m, _lib.stream_handle(device),
        ))
    return outputs.view(groups * max_m, weight.n)


def w4a16_contiguous(
    inputs: torch.Tensor,
    weight: PreparedWeight,
    m_indices: torch.Tensor,
    *,
    outputs: torch.Tensor | None = None,
    enable_pdl: bool = False,
) -> torch.Tensor:
    """Contiguous (prefill) grouped GEMM: ``[m, K]`` with each expert's rows padded
    to 128 (zeroed), ``m_indices`` ``[m] int32`` (-1 padding) -> ``[m, N]``."""
    if not isinstance(inputs, torch.Tensor):
        raise TypeError(f"inputs must be a torch.Tensor, got {type(inputs).__name__}")
    _check_weight(weight, inputs.device)
    _check_activation(inputs, weight.k)
    if inputs.dim() != 2:
        raise ValueError(f"inputs must be 2D [m, K], got {inputs.dim()}D")
    if not isinstance(m_indices, torch.Tensor):
        raise TypeError(f"m_indices must be a torch.Tensor, got {type(m_indices).__name__}")
    if m_indices.dtype != torch.int32:
        m_indices = m_indices.to(torch.int32)
    if (m_indices.dim() != 1 or not m_indices.is_cuda or not m_indices.is_contiguous()
            or m_indices.numel() != inputs.size(0)):
        raise ValueError(f"m_indices must be contiguous CUDA int32 [{inputs.size(0)}]")
    if inputs.size(0) % 128:
        raise ValueError(f"contiguous m={inputs.size(0)} must be 128-aligned (per-expert padded)")
    if not isinstance(enable_pdl, bool):
        raise TypeError(f"enable_pdl must be a bool, got {type(enable_pdl).__name__}")

    device = inputs.device
    m = inputs.size(0)
    if outputs is None:
        outputs = torch.empty((m, weight.n), dtype=torch.bfloat16, device=device)
    else:
        _check_outputs(outputs, (m, weight.n), device)
    lib = _lib.load()
    with torch.cuda.device(device):
        locks, workspace, ws_bytes = gemm_scratch(device, 256, None)
        _lib.check(lib.chord_b200_contiguous(
            inputs.data_ptr(), weight.packed.data_ptr(), weight.scale.data_ptr(),
            m_indices.data_ptr(), outputs.data_ptr(), locks.data_ptr(), locks.numel(),
            workspace.data_ptr(), ws_bytes, status_word(device).data_ptr(),
            m, weight.n, weight.k, weight.num_experts, _lib.stream_handle(device),
        ))
    return outputs.view(m, weight.n)


def masked(activation, weight, masked_m, expected_m: int, *, outputs=None, enable_pdl: bool = False):
    """Grouped masked (decode) GEMM.

    ``activation`` is BF16 ``[G, max_m, K]`` (or flat ``[G*max_m, K]``), ``weight``
    comes from ``pack_w4a16``, ``masked_m`` is the valid row count per expert
    ``[G] int32`` and ``expected_m`` its typical value.  Returns flat
    ``[G*max_m, N]``.  Same signature as chord_kernels/ops.py:49-69.
    """
    return w4a16_masked(activation, weight, masked_m, expected_m, outputs=outputs,
                        enable_pdl=enable_pdl)


def contiguous(activation, weight, m_indices, *, outputs=None, enable_pdl: bool = False):
    """Grouped contiguous (prefill) GEMM.

    ``activation`` is BF16 ``[m, K]`` with each expert's rows padded to a 128-row
    boundary (padding zeroed); ``m_indices`` ``[m] int32`` names each row's expert
    (-1 for padding).  Returns ``[m, N]``.  Same signature as
    chord_kernels/ops.py:72-90.
    """
    return w4a16_contiguous(activation, weight, m_indices, outputs=outputs, enable_pdl=enable_pdl)


__all__ = ["contiguous", "masked", "w4a16_contiguous", "w4a16_masked", "masked_tile_m"]
