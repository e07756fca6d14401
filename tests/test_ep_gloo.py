"""Expert-parallel dispatch/combine on two CPU ranks (gloo): the index arithmetic of
chord_b200.ep with the oracle standing in for the local GPU experts."""

import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _reference_layer(x, topk, codes13, scale13, codes2, scale2):
    """Single-process result: gate_up -> SiLU*mul -> down per route (FP32 accumulate)."""
    from oracle import w4a16_oracle as O

    top_k = topk.size(1)
    gate_up = O.reference_indexed(x, codes13, scale13, topk, top_k).to(torch.bfloat16)
    hidden = O.silu_mul(gate_up)
    down = O.reference_indexed(hidden, codes2, scale2, topk, top_k, projection="down")
    return down.to(torch.bfloat16).view(-1, top_k, codes2.size(1))


def _worker(rank, world, port, tmp):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from chord_b200 import ep
        from oracle import w4a16_oracle as O
        from tests.cases import make_weights

        experts_total, hidden, inter, tokens, top_k = 8, 128, 64, 12, 3
        codes13, scale13 = make_weights(experts_total, 2 * inter, hidden, 1)
        codes2, scale2 = make_weights(experts_total, hidden, inter, 2)
        g = torch.Generator().manual_seed(5)
        x_all = torch.randn((world * tokens, hidden), generator=g).to(torch.bfloat16)
        topk_all = O.topk_ids_random(world * tokens, top_k, experts_total, g)
        x = x_all[rank * tokens:(rank + 1) * tokens]
        topk = topk_all[rank * tokens:(rank + 1) * tokens]
        per_rank = experts_total // world
        lo = rank * per_rank

        def local_experts(rows, local_ids):
            ids = local_ids.view(-1, 1).to(torch.int32)
            assert ((ids >= 0) & (ids < per_rank)).all()
            gate_up = O.reference_indexed(rows, codes13[lo:lo + per_rank], scale13[lo:lo + per_rank],
                                          ids, 1).to(torch.bfloat16)
            h = O.silu_mul(gate_up)
            return O.reference_indexed(h, codes2[lo:lo + per_rank], scale2[lo:lo + per_rank],
                                       ids, 1, projection="down").to(torch.bfloat16)

        out = ep.moe_layer(x, topk, experts_total, local_experts, group=dist.group.WORLD)
        want = _reference_layer(x_all, topk_all, codes13, scale13, codes2, scale2)
        want = want[rank * tokens:(rank + 1) * tokens]
        torch.save({"equal": bool(torch.equal(out, want)), "shape": tuple(out.shape)},
                   os.path.join(tmp, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_rank_dispatch_combine_matches_single_process(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for rank in range(world):
        result = torch.load(tmp_path / f"rank{rank}.pt")
        assert result["shape"] == (12, 3, 128)
        assert result["equal"], f"rank {rank} differs from the single-process result"


def test_plan_groups_routes_by_owner():
    from chord_b200 import ep

    topk = torch.tensor([[0, 5], [7, 2], [4, 3], [1, 6]], dtype=torch.int32)
    plan = ep.plan_dispatch(topk, 8, 2)
    assert plan.send_counts == [4, 4] and plan.num_routes == 8 and plan.top_k == 2
    flat = topk.reshape(-1)
    assert (flat[plan.send_order[:4]] < 4).all() and (flat[plan.send_order[4:]] >= 4).all()
    assert torch.equal(plan.send_local_expert, (flat[plan.send_order] % 4).to(torch.int32))
    # stable: route order is kept inside a destination
    assert plan.send_order[:4].tolist() == sorted(plan.send_order[:4].tolist())
    with pytest.raises(ValueError):
        ep.plan_dispatch(topk, 8, 3)


def test_single_rank_layer_needs_no_process_group():
    from chord_b200 import ep

    x = torch.arange(12, dtype=torch.float32).view(4, 3)
    topk = torch.tensor([[1, 0], [0, 1], [1, 1], [0, 0]], dtype=torch.int32)
    out = ep.moe_layer(x, topk, 2, lambda rows, ids: rows * (ids.view(-1, 1).float() + 1))
    want = x.repeat_interleave(2, 0) * (topk.reshape(-1, 1).float() + 1)
    assert torch.equal(out, want.view(4, 2, 3))


def test_exchange_layout_covers_the_worst_case():
    """Buffer layout of the peer-memory exchange: the receive buffers hold every route of
    every rank (the worst case: all of them land on one rank) with every local expert's
    rows padded to whole routing blocks, regions are 256-byte aligned and do not overlap."""
    from chord_b200.ep import ExchangeLayout

    lay = ExchangeLayout.build(world=8, max_tokens=512, top_k=8, hidden_in=7168, hidden_out=7168,
                               state_bytes=17160, experts_per_rank=48, block_m=128)
    assert lay.routed_rows == 4096
    assert lay.capacity % 128 == 0 and 0 <= lay.capacity - (8 * 4096 + 48 * 127) < 128
    regions = [(lay.state, 17160), (lay.recv_tag, lay.capacity * 4),
               (lay.recv_x, lay.capacity * 7168 * 2), (lay.routed, lay.routed_rows * 7168 * 2)]
    end = 0
    for start, size in regions:
        assert start % 256 == 0 and start >= end
        end = start + size
    assert lay.total >= end
