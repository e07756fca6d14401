"""``masked`` / ``contiguous`` grouped W4A16 GEMMs, same interface as
chord_kernels/ops.py:49-90 and chord_kernels/operator/grouped/api.py:116-271.

The reference implements these for SM90 only (WGMMA); here they run on the same
sm_100a tcgen05 kernel as ``indexed`` with a different tile scheduler."""

from __future__ import annotations

import torch

from . import _checks, _lib
from .indexed_gemm import gemm_scratch, status_word
from .packing import PreparedWeight


def _operands(inputs, weight):
    """The checks `masked` and `contiguous` share (chord_kernels/operator/grouped/api.py:24-73;
    its SM90 gate and BLOCK_K rule do not apply here: K % 64 is all this kernel needs)."""
    _checks.tensor("inputs", inputs, cuda=False, contiguous=False)
    if not isinstance(weight, PreparedWeight):
        raise TypeError("weight must be a PreparedWeight from pack_w4a16()")
    if inputs.is_cuda:
        _checks.supported_gpu(inputs.device)
    _checks.prepared_weight(weight, inputs.device, dtype_error=TypeError)
    _checks.tensor("inputs", inputs, dtype=torch.bfloat16, nonempty=True)
    if inputs.size(-1) != weight.k:
        raise ValueError(f"inputs K={inputs.size(-1)} != weight K={weight.k}")


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
    _operands(inputs, weight)
    groups = weight.num_experts
    if inputs.dim() == 2:
        if inputs.size(0) % groups:
            raise ValueError(
                f"flat inputs rows {inputs.size(0)} are not divisible by num_experts={groups}")
        grouped = inputs.view(groups, inputs.size(0) // groups, weight.k)
    elif inputs.dim() == 3:
        if inputs.size(0) != groups:
            raise ValueError(f"inputs groups {inputs.size(0)} != num_experts={groups}")
        grouped = inputs
    else:
        raise ValueError(f"inputs must be 2D or 3D, got {inputs.dim()}D")
    _checks.tensor("masked_m", masked_m, cuda=False, contiguous=False)
    if masked_m.dtype != torch.int32:
        masked_m = masked_m.to(torch.int32)  # other integer types are cast, as in the reference
    if (masked_m.dim() != 1 or masked_m.numel() != groups or not masked_m.is_cuda
            or not masked_m.is_contiguous()):
        raise ValueError(f"masked_m must be contiguous CUDA int32 [{groups}]")
    _checks.integer("expected_m", expected_m, minimum=1, type_error=True)
    _checks.flag("enable_pdl", enable_pdl)

    device = inputs.device
    max_m = grouped.size(1)
    if outputs is None:
        outputs = torch.empty((groups * max_m, weight.n), dtype=torch.bfloat16, device=device)
    else:
        _checks.bf16_output(outputs, (groups * max_m, weight.n), device, exact_shape=False)
    tile_m = masked_tile_m(expected_m)
    lib = _lib.load()
    with _lib.on_device(device):
        locks, workspace, ws_bytes = gemm_scratch(device, tile_m, None)
        _lib.check(lib.chord_b200_masked(
            grouped.data_ptr(), weight.packed.data_ptr(), weight.scale.data_ptr(),
            masked_m.data_ptr(), outputs.data_ptr(), locks.data_ptr(), locks.numel(),
            workspace.data_ptr(), ws_bytes, status_word(device).data_ptr(),
            groups, max_m, weight.n, weight.k, tile_m, int(enable_pdl), _lib.stream_handle(device),
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
    _operands(inputs, weight)
    if inputs.dim() != 2:
        raise ValueError(f"inputs must be 2D [m, K], got {inputs.dim()}D")
    _checks.tensor("m_indices", m_indices, cuda=False, contiguous=False)
    if m_indices.dtype != torch.int32:
        m_indices = m_indices.to(torch.int32)
    if (m_indices.dim() != 1 or not m_indices.is_cuda or not m_indices.is_contiguous()
            or m_indices.numel() != inputs.size(0)):
        raise ValueError(f"m_indices must be contiguous CUDA int32 [{inputs.size(0)}]")
    if inputs.size(0) % 128:
        raise ValueError(f"contiguous m={inputs.size(0)} must be 128-aligned (per-expert padded)")
    _checks.flag("enable_pdl", enable_pdl)

    device = inputs.device
    m = inputs.size(0)
    if outputs is None:
        outputs = torch.empty((m, weight.n), dtype=torch.bfloat16, device=device)
    else:
        _checks.bf16_output(outputs, (m, weight.n), device, exact_shape=False)
    lib = _lib.load()
    with _lib.on_device(device):
        locks, workspace, ws_bytes = gemm_scratch(device, 256, None)
        _lib.check(lib.chord_b200_contiguous(
            inputs.data_ptr(), weight.packed.data_ptr(), weight.scale.data_ptr(),
            m_indices.data_ptr(), outputs.data_ptr(), locks.data_ptr(), locks.numel(),
            workspace.data_ptr(), ws_bytes, status_word(device).data_ptr(),
            m, weight.n, weight.k, weight.num_experts, int(enable_pdl), _lib.stream_handle(device),
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
