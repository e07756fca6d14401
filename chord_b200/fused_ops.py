"""The steps a serving engine runs either side of the expert GEMMs: SiLU*mul
between gate_up and down, and ``moe_align_block_size``.  The reference leaves
both to its caller (docs/getting_started.md:5-14) and its tests use a Python loop
for the alignment (tests/generators.py:192-230)."""

from __future__ import annotations

import torch

from . import _lib


def silu_mul(gate_up: torch.Tensor, *, sorted_ids: torch.Tensor | None = None,
             num_tokens_padded: torch.Tensor | None = None,
             outputs: torch.Tensor | None = None) -> torch.Tensor:
    """``out[r, j] = silu(gate_up[r, j]) * gate_up[r, I + j]`` (gate columns first).

    With ``sorted_ids`` / ``num_tokens_padded`` only the rows the routing names are
    computed: the rows ``indexed`` wrote."""
    if not isinstance(gate_up, torch.Tensor) or gate_up.dtype != torch.bfloat16 or gate_up.ndim != 2:
        raise TypeError("gate_up must be a 2D torch.bfloat16 tensor")
    if not gate_up.is_cuda or not gate_up.is_contiguous():
        raise ValueError("gate_up must be a contiguous CUDA tensor")
    rows, width = gate_up.shape
    if width % 16:
        raise ValueError(f"gate_up width must be divisible by 16, got {width}")
    inter = width // 2
    device = gate_up.device
    if outputs is None:
        outputs = torch.empty((rows, inter), dtype=torch.bfloat16, device=device)
    elif (outputs.dtype != torch.bfloat16 or tuple(outputs.shape) != (rows, inter)
          or not outputs.is_contiguous() or outputs.device != device):
        raise ValueError(f"outputs must be contiguous BF16 {(rows, inter)} on {device}")
    lib = _lib.load()
    with _lib.on_device(device):
        stream = _lib.stream_handle(device)
        if sorted_ids is None:
            _lib.check(lib.chord_b200_silu_mul(gate_up.data_ptr(), outputs.data_ptr(), rows, inter, stream))
        else:
            if num_tokens_padded is None:
                raise ValueError("num_tokens_padded is required with sorted_ids")
            _lib.check(lib.chord_b200_silu_mul_routed(
                gate_up.data_ptr(), outputs.data_ptr(), sorted_ids.data_ptr(), sorted_ids.numel(),
                num_tokens_padded.data_ptr(), rows, inter, stream,
            ))
    return outputs


def moe_align_block_size(topk_ids: torch.Tensor, block_m: int, num_experts: int, *,
                         expert_base: int = 0):
    """Sort routes by expert into ``block_m`` blocks padded with the sentinel
    ``topk_ids.numel()``.  Returns ``(sorted_ids, expert_ids, num_tokens_padded)``
    in the contract ``indexed`` consumes; buffers are worst-case sized and only the
    first ``num_tokens_padded`` ids / ``num_tokens_padded // block_m`` experts are
    meaningful.  Only routes to experts in ``[expert_base, expert_base + num_experts)``
    are kept, and ``expert_ids`` holds local indices (expert parallelism)."""
    if not isinstance(topk_ids, torch.Tensor) or topk_ids.dtype != torch.int32:
        raise TypeError("topk_ids must be a torch.int32 tensor")
    if not topk_ids.is_cuda or not topk_ids.is_contiguous():
        raise ValueError("topk_ids must be a contiguous CUDA tensor")
    if isinstance(block_m, bool) or not isinstance(block_m, int) or block_m <= 0 or block_m % 8:
        raise ValueError(f"block_m must be a positive multiple of 8, got {block_m!r}")
    device = topk_ids.device
    numel = topk_ids.numel()
    worst = min(numel + num_experts * (block_m - 1), numel * block_m)
    blocks = max(worst // block_m, 1)
    sorted_ids = torch.empty(blocks * block_m, dtype=torch.int32, device=device)
    expert_ids = torch.empty(blocks, dtype=torch.int32, device=device)
    num_tokens_padded = torch.empty(1, dtype=torch.int32, device=device)
    lib = _lib.load()
    with _lib.on_device(device):
        _lib.check(lib.chord_b200_moe_align_block_size(
            topk_ids.data_ptr(), numel, expert_base, num_experts, block_m,
            sorted_ids.data_ptr(), sorted_ids.numel(), expert_ids.data_ptr(), expert_ids.numel(),
            num_tokens_padded.data_ptr(), _lib.stream_handle(device),
        ))
    return sorted_ids, expert_ids, num_tokens_padded


__all__ = ["moe_align_block_size", "silu_mul"]
