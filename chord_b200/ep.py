"""Expert-parallel MoE layer around the local W4A16 expert GEMMs.

The reference library stops at the per-rank GEMMs: "EP8" only selects per-GPU
shapes and its routing "may carry only this rank's routes"
(docs/getting_started.md:21, tests/generators.py:400-423); it has no
communication code.  This module adds the exchange a deployment needs around
them: experts are split contiguously over the ranks of one node, tokens are
dispatched to the ranks that own their experts with ``all_to_all_single`` (NCCL
over NVLink on GPUs, gloo in the CPU tests), the local ``indexed`` gate_up ->
SiLU*mul -> ``indexed`` down runs on what arrived, and the results travel back
the same way.  With one rank every collective is skipped.

The index arithmetic (who sends what where, and how results find their way back)
is plain torch and runs on CPU tensors too, so it is tested with two gloo ranks
without a GPU.
"""

from __future__ import annotations

import dataclasses
from typing import Callable

import torch
import torch.distributed as dist


@dataclasses.dataclass
class DispatchPlan:
    """Where every route of this rank's tokens goes.

    ``send_order[i]`` is the route (``token * top_k + slot``) travelling in send
    position ``i``; positions are grouped by destination rank, ``send_counts[r]``
    of them to rank ``r``.  ``send_local_expert[i]`` is the expert's index on its
    owner.
    """

    send_order: torch.Tensor         # int64 [routes]
    send_counts: list[int]           # per destination rank
    send_local_expert: torch.Tensor  # int32 [routes]
    num_routes: int
    top_k: int


def plan_dispatch(topk_ids: torch.Tensor, num_experts_total: int, world_size: int) -> DispatchPlan:
    """Group this rank's routes by the rank that owns their expert (experts are split
    contiguously: rank r owns ``[r * E/R, (r + 1) * E/R)``)."""
    if num_experts_total % world_size:
        raise ValueError(
            f"num_experts_total={num_experts_total} is not divisible by world_size={world_size}")
    experts_per_rank = num_experts_total // world_size
    flat = topk_ids.reshape(-1).to(torch.int64)
    dest = torch.div(flat, experts_per_rank, rounding_mode="floor")
    # Stable sort keeps routes of one destination in route order, which makes the
    # whole exchange deterministic.
    send_order = torch.sort(dest, stable=True).indices
    counts = torch.bincount(dest, minlength=world_size)
    return DispatchPlan(
        send_order=send_order,
        send_counts=[int(c) for c in counts.cpu().tolist()],
        send_local_expert=(flat[send_order] % experts_per_rank).to(torch.int32),
        num_routes=flat.numel(),
        top_k=topk_ids.size(-1) if topk_ids.ndim > 1 else 1,
    )


def exchange_counts(send_counts: list[int], group, device) -> list[int]:
    """Tell every rank how many rows to expect from every other rank."""
    world_size = dist.get_world_size(group) if group is not None else 1
    if world_size == 1:
        return list(send_counts)
    send = torch.tensor(send_counts, dtype=torch.int64, device=device)
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return [int(c) for c in recv.cpu().tolist()]


def all_to_all_rows(rows: torch.Tensor, send_counts: list[int], recv_counts: list[int], group):
    """Uneven all-to-all of the leading dimension."""
    world_size = dist.get_world_size(group) if group is not None else 1
    if world_size == 1:
        return rows
    out = rows.new_empty((sum(recv_counts),) + tuple(rows.shape[1:]))
    dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=recv_counts,
                           input_split_sizes=send_counts, group=group)
    return out


def moe_layer(
    x: torch.Tensor,
    topk_ids: torch.Tensor,
    num_experts_total: int,
    local_experts: Callable[[torch.Tensor, torch.Tensor], torch.Tensor],
    group=None,
) -> torch.Tensor:
    """Routed expert outputs ``[tokens, top_k, hidden_out]`` for this rank's tokens.

    ``x`` is ``[tokens, hidden]`` and ``topk_ids`` ``[tokens, top_k]`` (global
    expert ids).  ``local_experts(rows, local_expert_ids)`` computes, on the owner
    rank, one output row per received row; on GPUs it is :func:`local_expert_mlp`.
    The top-k weighting and the sum over ``top_k`` are left to the caller, as in the
    reference (docs/getting_started.md:20).
    """
    world_size = dist.get_world_size(group) if (group is not None or dist.is_initialized()) else 1
    if world_size == 1:
        group = None
    plan = plan_dispatch(topk_ids, num_experts_total, world_size)
    tokens_of_route = torch.div(plan.send_order, plan.top_k, rounding_mode="floor")
    send_rows = x.index_select(0, tokens_of_route.to(x.device))
    recv_counts = exchange_counts(plan.send_counts, group, x.device)
    recv_rows = all_to_all_rows(send_rows, plan.send_counts, recv_counts, group)
    recv_experts = all_to_all_rows(plan.send_local_expert.to(x.device), plan.send_counts,
                                   recv_counts, group)
    out_rows = local_experts(recv_rows, recv_experts)
    back = all_to_all_rows(out_rows, recv_counts, plan.send_counts, group)
    routed = back.new_empty((plan.num_routes, back.size(-1)))
    routed.index_copy_(0, plan.send_order.to(back.device), back)
    return routed.view(-1, plan.top_k, back.size(-1))


def local_expert_mlp(w13, w2, *, locks=None):
    """``local_experts`` callback for :func:`moe_layer` on a GPU: routing alignment,
    ``indexed`` gate_up, SiLU*mul on the routed rows, ``indexed`` down.

    ``w13`` / ``w2`` are the :class:`PreparedWeight` of this rank's experts.  Every
    received row is one route, so both GEMMs run with ``top_k=1``.
    """
    from .fused_ops import moe_align_block_size, silu_mul
    from .indexed_gemm import indexed, select_block_m

    num_local = w13.num_experts

    def run(rows: torch.Tensor, local_expert_ids: torch.Tensor) -> torch.Tensor:
        count = rows.size(0)
        hidden_out = w2.n
        if count == 0:
            return rows.new_empty((0, hidden_out))
        block_m = select_block_m(w13.n, w13.k, num_local, count)
        sorted_ids, expert_ids, padded = moe_align_block_size(
            local_expert_ids.contiguous().view(-1, 1), block_m, num_local)
        gate_up = indexed(rows, w13, sorted_ids, expert_ids, padded, 1, locks=locks,
                          block_m=block_m)
        hidden = silu_mul(gate_up, sorted_ids=sorted_ids, num_tokens_padded=padded)
        return indexed(hidden, w2, sorted_ids, expert_ids, padded, 1, locks=locks,
                       block_m=block_m)

    return run


__all__ = ["DispatchPlan", "local_expert_mlp", "moe_layer", "plan_dispatch"]
