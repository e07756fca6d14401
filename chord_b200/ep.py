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

Two forms of the exchange live here.  :func:`moe_layer` does it with
``all_to_all_single`` and plain torch index arithmetic; it runs on CPU tensors too and
is what the two-rank gloo tests exercise.  :class:`ExpertParallelLayer` is the form for
GPUs of one NVSwitch domain: the library's own kernels move the rows through peer
memory (csrc/ep.cu) - dispatch by 16-byte peer stores into the owner's receive
buffer, combine by the down projection's epilogue storing every result row straight
into the result tensor of the GPU the token came from - with no collective call and
no host synchronisation on the path.
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


# ------------------------------------------------- exchange over peer memory --

def _align(value: int, unit: int = 256) -> int:
    return (value + unit - 1) // unit * unit


@dataclasses.dataclass(frozen=True)
class ExchangeLayout:
    """Byte offsets of one rank's exchange buffers inside its peer-visible allocation."""

    capacity: int        # slots of the receive buffers: every route of every rank, each local expert's rows padded to whole routing blocks
    routed_rows: int     # rows of this rank's result tensor (tokens * top_k)
    hidden_in: int
    hidden_out: int
    state: int
    recv_tag: int
    recv_x: int
    routed: int
    total: int

    @staticmethod
    def build(world: int, max_tokens: int, top_k: int, hidden_in: int, hidden_out: int,
              state_bytes: int, experts_per_rank: int = 0, block_m: int = 1) -> "ExchangeLayout":
        routed_rows = max_tokens * top_k
        # the worst case: every route lands on one rank, every expert's last block nearly empty
        worst = world * routed_rows + experts_per_rank * (block_m - 1)
        capacity = (worst + block_m - 1) // block_m * block_m
        state = 0
        recv_tag = _align(state + state_bytes)
        recv_x = _align(recv_tag + capacity * 4)
        routed = _align(recv_x + capacity * hidden_in * 2)
        total = _align(routed + routed_rows * hidden_out * 2)
        return ExchangeLayout(capacity, routed_rows, hidden_in, hidden_out, state, recv_tag, recv_x,
                              routed, total)


class SymmetricFabric:
    """One peer-visible allocation per rank, mapped into every process of ``group`` with
    torch's symmetric memory (plain peer mappings; multicast binding is switched off
    because these kernels use ordinary loads and stores only)."""

    def __init__(self, nbytes: int, group, device: torch.device):
        import os

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.buffer = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        self.buffer.zero_()
        self.handle = symm_mem.rendezvous(self.buffer, group)
        self.base = [int(p) for p in self.handle.buffer_ptrs]
        torch.cuda.synchronize(device)
        dist.barrier(group)                 # every rank's state is zero before anyone writes


class LocalFabric:
    """All ranks inside one process on one GPU (tests): one ordinary allocation per rank."""

    def __init__(self, nbytes: int, world: int, device: torch.device):
        self.world = world
        self.buffers = [torch.zeros(nbytes, dtype=torch.uint8, device=device) for _ in range(world)]
        self.base = [b.data_ptr() for b in self.buffers]

    def view(self, rank: int) -> "LocalFabric":
        clone = object.__new__(LocalFabric)
        clone.world, clone.buffers, clone.base = self.world, self.buffers, self.base
        clone.rank, clone.buffer = rank, self.buffers[rank]
        return clone


class ExpertParallelLayer:
    """gate_up -> SiLU*mul -> down of a Mixture-of-Experts layer whose experts are split
    contiguously over the ranks of ``fabric`` (rank r owns experts
    ``[r * E / R, (r + 1) * E / R)``), with the token exchange done by this library's
    kernels over peer memory.

    ``layer(x, topk_ids)`` takes this rank's tokens ``x [tokens, hidden]`` and their
    global expert ids ``topk_ids [tokens, top_k]`` (int32) and returns the routed expert
    outputs ``[tokens, top_k, hidden_out]``; top-k weighting and the sum over ``top_k``
    are left to the caller, as in the reference (docs/getting_started.md:20).  Every rank
    must call it the same number of times (the calls pair up across ranks), on one
    stream, and read the result before its next call (the result tensor is reused).

    The steps are separate methods (``plan``, ``dispatch``, ``local_experts``,
    ``finish``) so that a test can run several ranks on one GPU by doing each step for
    all ranks before the next: a kernel then never waits for a later launch.
    With one rank there is no exchange: the routing is aligned and the two GEMMs run on
    the tokens directly.
    """

    @staticmethod
    def exchange_layout(w13, w2, *, world: int, max_tokens: int, top_k: int) -> "ExchangeLayout":
        """Layout of one rank's peer-visible buffers (what a fabric has to allocate): the
        receive buffers are sized in routing blocks of the block size the local GEMMs use."""
        from . import _lib
        from .indexed_gemm import select_block_m

        # expected rows per rank if the routes spread evenly: sizes the routing blocks
        block_m = select_block_m(w13.n, w13.k, w13.num_experts, max_tokens * top_k)
        return ExchangeLayout.build(world, max_tokens, top_k, w13.k, w2.n,
                                    _lib.load().chord_b200_ep_state_bytes(), w13.num_experts, block_m)

    def __init__(self, w13, w2, *, num_experts_total: int, max_tokens: int, top_k: int,
                 fabric=None, group=None):
        from . import _lib

        self.lib = _lib.load()
        self.w13, self.w2 = w13, w2
        self.device = w13.packed.device
        self.top_k, self.max_tokens = top_k, max_tokens
        self.hidden_in, self.hidden_out, self.inter2 = w13.k, w2.n, w13.n
        if w2.k * 2 != w13.n:
            raise ValueError(f"w13 has {w13.n} rows, w2 reduces over {w2.k}: expected n13 == 2 * k2")
        if fabric is None and group is not None and dist.get_world_size(group) > 1:
            layout = self.exchange_layout(w13, w2, world=dist.get_world_size(group), max_tokens=max_tokens,
                                          top_k=top_k)
            fabric = SymmetricFabric(layout.total, group, self.device)
        self.fabric = fabric
        self.world = fabric.world if fabric is not None else 1
        self.rank = fabric.rank if fabric is not None else 0
        if num_experts_total % self.world or num_experts_total // self.world != w13.num_experts:
            raise ValueError(
                f"{num_experts_total} experts over {self.world} ranks need {num_experts_total // self.world} "
                f"local experts, the weights hold {w13.num_experts}")
        self.experts_per_rank = w13.num_experts
        self.locks = torch.zeros(1024, dtype=torch.int32, device=self.device)
        self.epoch = 0
        self.spans = None          # optional: list that receives (name, start event, end event)
        if self.world == 1:
            return
        self.layout = self.exchange_layout(w13, w2, world=self.world, max_tokens=max_tokens, top_k=top_k)
        lay, dev = self.layout, self.device
        if fabric.buffer.numel() < lay.total:
            raise ValueError("the fabric's allocation is smaller than the exchange layout")

        def table(offset):
            return torch.tensor([b + offset for b in fabric.base], dtype=torch.int64, device=dev)

        self.peer_state, self.peer_recv_tag = table(lay.state), table(lay.recv_tag)
        self.peer_recv_x, self.peer_routed = table(lay.recv_x), table(lay.routed)
        buf = fabric.buffer
        self.state = buf[lay.state:lay.recv_tag]
        self.recv_tag = buf[lay.recv_tag:lay.recv_tag + lay.capacity * 4].view(torch.int32)
        self.recv_x = buf[lay.recv_x:lay.recv_x + lay.capacity * self.hidden_in * 2].view(
            torch.bfloat16).view(lay.capacity, self.hidden_in)
        self.routed = buf[lay.routed:lay.routed + lay.routed_rows * self.hidden_out * 2].view(
            torch.bfloat16).view(lay.routed_rows, self.hidden_out)
        from .indexed_gemm import select_block_m

        self.block_m = select_block_m(w13.n, w13.k, self.experts_per_rank, lay.routed_rows)
        blocks = lay.capacity // self.block_m
        self.sorted_ids = torch.empty(lay.capacity, dtype=torch.int32, device=dev)
        self.expert_ids = torch.empty(blocks, dtype=torch.int32, device=dev)
        self.padded = torch.zeros(1, dtype=torch.int32, device=dev)
        self.recv_count = torch.zeros(1, dtype=torch.int32, device=dev)
        self.send_pos = torch.empty(lay.routed_rows, dtype=torch.int32, device=dev)
        self.row_ptr = torch.zeros(lay.capacity, dtype=torch.int64, device=dev)
        self.hidden = torch.empty((lay.capacity, self.inter2 // 2), dtype=torch.bfloat16, device=dev)
        fused = bool(self.lib.chord_b200_gate_up_silu_supported(w13.n, w13.k, self.block_m))
        self.gate_up = None if fused else torch.empty((lay.capacity, self.inter2), dtype=torch.bfloat16,
                                                      device=dev)

    # -- helpers ---------------------------------------------------------------------
    def _stream(self):
        from . import _lib

        return _lib.stream_handle(self.device)

    def _span(self, name):
        if self.spans is None:
            return None
        start = torch.cuda.Event(enable_timing=True)
        start.record()
        return name, start

    def _end(self, span):
        if span is not None:
            stop = torch.cuda.Event(enable_timing=True)
            stop.record()
            self.spans.append((span[0], span[1], stop))

    def status(self) -> int:
        """Bits of bounded cross-GPU waits that ran out (0 = none); synchronises."""
        if self.world == 1:
            return 0
        torch.cuda.synchronize(self.device)
        end = self.lib.chord_b200_ep_state_bytes()      # the status word closes the state
        return int(self.state[end - 4:end].view(torch.int32).item())

    # -- the steps of one call -------------------------------------------------------
    def plan(self, x: torch.Tensor, topk_ids: torch.Tensor) -> None:
        from . import _lib

        if topk_ids.dtype != torch.int32 or not topk_ids.is_contiguous():
            raise TypeError("topk_ids must be a contiguous torch.int32 tensor")
        if x.dtype != torch.bfloat16 or not x.is_contiguous() or x.size(1) != self.hidden_in:
            raise ValueError(f"x must be contiguous BF16 [tokens, {self.hidden_in}]")
        tokens = x.size(0)
        if tokens > self.max_tokens or topk_ids.numel() != tokens * self.top_k:
            raise ValueError(f"at most {self.max_tokens} tokens with {self.top_k} expert ids each")
        self.epoch += 1
        self._x, self._topk, self._routes = x, topk_ids, tokens * self.top_k
        span = self._span("plan")
        _lib.check(self.lib.chord_b200_ep_plan(
            topk_ids.data_ptr(), self._routes, self.experts_per_rank, self.world, self.rank,
            self.send_pos.data_ptr(), self.peer_state.data_ptr(), self.epoch, self._stream()))
        self._end(span)

    def dispatch(self) -> None:
        from . import _lib

        span = self._span("dispatch")
        _lib.check(self.lib.chord_b200_ep_dispatch(
            self._x.data_ptr(), self._topk.data_ptr(), self.send_pos.data_ptr(), self._routes, self.top_k,
            self.hidden_in, self.experts_per_rank, self.world, self.rank, self.state.data_ptr(),
            self.peer_state.data_ptr(), self.peer_recv_x.data_ptr(), self.peer_recv_tag.data_ptr(),
            self.layout.capacity, self.block_m, self.epoch, self._stream()))
        self._end(span)

    def local_experts(self) -> None:
        from . import _lib
        from .indexed_gemm import gemm_scratch, status_word

        lay = self.layout
        span = self._span("align")
        _lib.check(self.lib.chord_b200_ep_align(
            self.state.data_ptr(), self.recv_tag.data_ptr(), lay.capacity, self.world, self.rank,
            self.experts_per_rank, self.block_m, self.sorted_ids.data_ptr(), self.sorted_ids.numel(),
            self.expert_ids.data_ptr(), self.expert_ids.numel(), self.padded.data_ptr(),
            self.recv_count.data_ptr(), self.peer_routed.data_ptr(), lay.routed_rows, self.hidden_out,
            self.row_ptr.data_ptr(), self.epoch, self._stream()))
        self._end(span)
        span = self._span("experts")
        # The rows arrived in routing-slot order: both GEMMs load them where they are.
        # gate_up with SiLU*mul in the epilogue (a separate SiLU*mul where that is not
        # supported), then down, whose epilogue stores every result row straight into the
        # result tensor of the rank the token came from.
        from .fused_ops import silu_mul

        status = status_word(self.device).data_ptr()

        def slots_gemm(weight, x, out_ptr, rows_ptr, fuse):
            locks, workspace, ws_bytes = gemm_scratch(self.device, self.block_m, self.locks,
                                                      self.sorted_ids.numel(), weight.k)
            _lib.check(self.lib.chord_b200_indexed_slots(
                x.data_ptr(), weight.packed.data_ptr(), weight.scale.data_ptr(),
                self.sorted_ids.data_ptr(), self.sorted_ids.numel(), self.expert_ids.data_ptr(),
                self.expert_ids.numel(), self.padded.data_ptr(), out_ptr, rows_ptr,
                locks.data_ptr(), locks.numel(), workspace.data_ptr(), ws_bytes, status, lay.capacity,
                weight.n, weight.k, self.experts_per_rank, self.block_m, fuse, self._stream()))

        if self.gate_up is None:
            slots_gemm(self.w13, self.recv_x, self.hidden.data_ptr(), 0, 1)
        else:
            slots_gemm(self.w13, self.recv_x, self.gate_up.data_ptr(), 0, 0)
            silu_mul(self.gate_up, sorted_ids=self.sorted_ids, num_tokens_padded=self.padded,
                     outputs=self.hidden)
        slots_gemm(self.w2, self.hidden, 0, self.row_ptr.data_ptr(), 0)
        _lib.check(self.lib.chord_b200_ep_combine_signal(
            self.peer_state.data_ptr(), self.world, self.rank, self.epoch, self._stream()))
        self._end(span)

    def finish(self) -> torch.Tensor:
        from . import _lib

        span = self._span("combine_wait")
        _lib.check(self.lib.chord_b200_ep_combine_wait(
            self.state.data_ptr(), self.world, self.epoch, self._stream()))
        self._end(span)
        return self.routed[: self._routes].view(-1, self.top_k, self.hidden_out)

    def _single_rank(self, x, topk_ids):
        from .fused_ops import moe_align_block_size
        from .indexed_gemm import indexed, indexed_gate_up_silu, select_block_m

        span = self._span("experts")
        tokens = x.size(0)
        block_m = select_block_m(self.w13.n, self.w13.k, self.experts_per_rank, tokens * self.top_k)
        routing = moe_align_block_size(topk_ids, block_m, self.experts_per_rank)
        hidden = indexed_gate_up_silu(x, self.w13, *routing, self.top_k, locks=self.locks, block_m=block_m)
        out = indexed(hidden, self.w2, *routing, 1, locks=self.locks, block_m=block_m)
        self._end(span)
        return out.view(tokens, self.top_k, self.hidden_out)

    def __call__(self, x: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        with torch.cuda.device(self.device):
            if self.world == 1:
                return self._single_rank(x, topk_ids)
            self.plan(x, topk_ids)
            self.dispatch()
            self.local_experts()
            return self.finish()


__all__ = ["DispatchPlan", "ExchangeLayout", "ExpertParallelLayer", "LocalFabric", "SymmetricFabric",
           "local_expert_mlp", "moe_layer", "plan_dispatch"]
