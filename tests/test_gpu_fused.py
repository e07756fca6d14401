"""SiLU*mul, routing alignment and the single-GPU expert-parallel layer on the GPU."""

import pytest
import torch

from oracle import w4a16_oracle as O
from tests.cases import make_weights

pytestmark = pytest.mark.gpu


def test_silu_mul_matches_oracle(device):
    import chord_b200

    g = torch.Generator().manual_seed(5)
    gate_up = (torch.randn((37, 4096), generator=g) * 3).to(torch.bfloat16)
    got = chord_b200.silu_mul(gate_up.to(device)).cpu()
    want = O.silu_mul(gate_up)
    # fast exponential on the device: allow one BF16 ulp
    assert (got.float() - want.float()).abs().max() <= 2.0 ** -7 * want.float().abs().max()
    assert (got.view(torch.int16) != want.view(torch.int16)).float().mean() < 0.02


def test_silu_mul_routed_touches_only_routed_rows(device):
    import chord_b200

    g = torch.Generator().manual_seed(6)
    gate_up = torch.randn((64, 512), generator=g).to(torch.bfloat16)
    topk = O.topk_ids_random(8, 8, 384, g)
    sorted_ids, _, padded = O.align_routing_blocks(topk, 16, 48, 0)
    out = torch.full((64, 256), float("nan"), dtype=torch.bfloat16, device=device)
    if sorted_ids.numel() == 0:
        pytest.skip("draw routed nothing locally")
    chord_b200.silu_mul(gate_up.to(device), sorted_ids=sorted_ids.to(device),
                        num_tokens_padded=padded.to(device).reshape(1), outputs=out)
    got = out.float().cpu()
    rows = sorted_ids[sorted_ids < 64].long()
    mask = torch.zeros(64, dtype=torch.bool)
    mask[rows] = True
    assert torch.equal(~torch.isnan(got).any(dim=1), mask)
    want = O.silu_mul(gate_up).float()
    assert (got[mask] - want[mask]).abs().max() <= 2.0 ** -7 * want.abs().max()


@pytest.mark.parametrize("tokens,top_k,total,local,base,block_m", [
    (64, 2, 8, 8, 0, 16), (256, 8, 384, 48, 96, 16), (4096, 8, 384, 384, 0, 64), (3, 8, 384, 48, 0, 8),
    (1, 8, 384, 48, 336, 16), (1000, 4, 64, 64, 0, 128), (0, 8, 384, 48, 0, 16),
])
def test_moe_align_block_size_bit_exact(device, tokens, top_k, total, local, base, block_m):
    import chord_b200

    g = torch.Generator().manual_seed(tokens + block_m)
    topk = O.topk_ids_random(tokens, top_k, total, g) if tokens else torch.zeros((0, top_k), dtype=torch.int32)
    s, e, p = chord_b200.moe_align_block_size(topk.to(device), block_m, local, expert_base=base)
    rs, re, rp = O.align_routing_blocks(topk, block_m, local, base)
    count = int(p.item())
    assert count == int(rp)
    assert torch.equal(s.cpu()[:count], rs)
    assert torch.equal(e.cpu()[: count // block_m], re)


def test_single_gpu_layer_matches_oracle(device):
    """The expert-parallel layer with one rank: alignment, gate_up, SiLU*mul, down."""
    import chord_b200
    from chord_b200 import ep

    experts, hidden, inter, tokens, top_k = 8, 512, 256, 40, 4
    codes13, scale13 = make_weights(experts, 2 * inter, hidden, 1)
    codes2, scale2 = make_weights(experts, hidden, inter, 2)
    g = torch.Generator().manual_seed(7)
    x = torch.randn((tokens, hidden), generator=g).to(torch.bfloat16)
    topk = O.topk_ids_random(tokens, top_k, experts, g)
    w13 = chord_b200.pack_w4a16(codes13.to(device), scale13.to(device))
    w2 = chord_b200.pack_w4a16(codes2.to(device), scale2.to(device))
    out = ep.moe_layer(x.to(device), topk.to(device), experts, ep.local_expert_mlp(w13, w2))
    assert out.shape == (tokens, top_k, hidden)
    gate_up = O.reference_indexed(x, codes13, scale13, topk, top_k).to(torch.bfloat16)
    ref = O.reference_indexed(O.silu_mul(gate_up), codes2, scale2, topk, top_k, projection="down")
    got = out.float().cpu().view(tokens * top_k, hidden)
    assert O.cosine_diff(got, ref) <= 5e-3
    assert O.max_abs_rel(got, ref) <= 2e-2      # two GEMMs and an activation in BF16


@pytest.mark.parametrize("world,tokens,top_k", [(2, 24, 2), (4, 33, 4), (2, 96, 4), (2, 300, 4)])
def test_peer_memory_exchange_with_all_ranks_on_one_gpu(device, world, tokens, top_k):
    """The expert-parallel layer's own kernels (plan, dispatch by peer stores, receive-side
    alignment, down projection storing into the source rank's result tensor, flags) with
    every rank living on this one GPU: each step is run for all ranks before the next, so
    no kernel waits for a later launch.  Every rank's routed outputs must equal the
    oracle's gate_up -> SiLU*mul -> down on the owning expert's weights.  The rows arrive
    in routing-slot order and the GEMMs load them in place; the cases cover routing blocks
    of 16 to 256 rows (both GEMM kernels)."""
    import chord_b200
    from chord_b200 import ep

    experts_total, hidden, inter = 8, 256, 128
    per_rank = experts_total // world
    codes13, scale13 = make_weights(experts_total, 2 * inter, hidden, seed=61)
    codes2, scale2 = make_weights(experts_total, hidden, inter, seed=62)
    weights = []
    for r in range(world):
        lo, hi = r * per_rank, (r + 1) * per_rank
        weights.append((chord_b200.pack_w4a16(codes13[lo:hi].to(device), scale13[lo:hi].to(device)),
                        chord_b200.pack_w4a16(codes2[lo:hi].to(device), scale2[lo:hi].to(device))))
    layout = ep.ExpertParallelLayer.exchange_layout(*weights[0], world=world, max_tokens=tokens, top_k=top_k)
    fabric = ep.LocalFabric(layout.total, world, device)
    layers, xs, topks = [], [], []
    g = torch.Generator().manual_seed(63)
    for r in range(world):
        w13, w2 = weights[r]
        layers.append(ep.ExpertParallelLayer(w13, w2, num_experts_total=experts_total, max_tokens=tokens,
                                             top_k=top_k, fabric=fabric.view(r)))
        n_tok = tokens - r                       # ranks bring different token counts
        xs.append(torch.randn((n_tok, hidden), generator=g).to(torch.bfloat16))
        topks.append(O.topk_ids_random(n_tok, top_k, experts_total, g))
    for call in range(2):                        # two calls: epochs advance, nothing is reset
        for r, layer in enumerate(layers):
            layer.plan(xs[r].to(device), topks[r].to(device))
        for layer in layers:
            layer.dispatch()
        for layer in layers:
            layer.local_experts()
        outs = [layer.finish().float().cpu() for layer in layers]
        for r, layer in enumerate(layers):
            assert layer.status() == 0
            n_tok = xs[r].size(0)
            gate_up = O.reference_indexed(xs[r], codes13, scale13, topks[r], top_k)
            hidden_rows = O.silu_mul(gate_up.to(torch.bfloat16))
            ref = O.reference_indexed(hidden_rows, codes2, scale2, topks[r], top_k, projection="down")
            got = outs[r].reshape(n_tok * top_k, hidden)
            assert not bool(torch.isnan(got).any())
            assert O.cosine_diff(got, ref) <= 5e-3
            assert O.max_abs_rel(got, ref) <= 2e-2   # two GEMMs and an activation, each rounded to BF16
        xs = [x * 0.5 for x in xs]               # new inputs for the second call


@pytest.mark.parametrize("experts,n,k,m,top_k,block_m", [
    (8, 512, 512, 24, 2, 16),       # decode kernel: gate and up block side by side in one worker
    (2, 256, 7168, 6, 1, 16),       # few tiles on many workers: every tile through the stream-K fix-up
    (6, 1024, 640, 300, 2, 128),    # general kernel, 128-row routing blocks (slot-ordered copy of the rows)
    (4, 512, 384, 200, 1, 64),      # general kernel, 64-row blocks
    (4, 512, 256, 40, 2, 32),       # no fused kernel for this block size: GEMM + SiLU*mul behind the same call
])
def test_gate_up_with_fused_silu_mul(device, experts, n, k, m, top_k, block_m):
    """`indexed_gate_up_silu` against the oracle's gate_up -> SiLU*mul: the fused kernels
    apply the activation to the FP32 accumulators (one rounding), so the comparison is
    against silu(gate) * up of the oracle's FP32 GEMM result."""
    import chord_b200
    from tests.cases import make_indexed_case

    case = make_indexed_case(num_experts=experts, n=n, k=k, m=m, top_k=top_k, block_m=block_m, seed=70 + m)
    w = chord_b200.pack_w4a16(case["codes"].to(device), case["scale"].to(device))
    routing = (case["sorted_ids"].to(device), case["expert_ids"].to(device),
               case["num_tokens_padded"].to(device).reshape(1))
    locks = torch.zeros(1024, dtype=torch.int32, device=device)
    out = torch.full((m * top_k, n // 2), float("nan"), dtype=torch.bfloat16, device=device)
    outs = []
    for _ in range(3):
        res = chord_b200.indexed_gate_up_silu(case["x"].to(device), w, *routing, top_k, locks=locks,
                                              outputs=out, block_m=block_m)
        outs.append(res.clone())
    chord_b200.check_status(device)
    assert bool((locks == 0).all())
    ref = O.reference_indexed(case["x"], case["codes"], case["scale"], case["topk_ids"], top_k)
    want = torch.nn.functional.silu(ref[:, : n // 2]) * ref[:, n // 2:]
    got = outs[0].float().cpu()
    assert not bool(torch.isnan(got).any())      # every route of this case is local
    assert O.cosine_diff(got, want) <= 5e-3
    assert O.max_abs_rel(got, want) <= 1.5e-2    # BF16 output of a product of two GEMM results
    for other in outs[1:]:
        assert torch.equal(other.view(torch.int16), outs[0].view(torch.int16))


@pytest.mark.parametrize("experts,n,k,m,block_m,fuse", [
    (6, 1024, 640, 500, 128, 0), (6, 1024, 640, 500, 128, 1), (4, 512, 2304, 700, 256, 0),
    (8, 512, 512, 40, 16, 0), (8, 512, 512, 40, 16, 1), (4, 512, 384, 150, 64, 1),
])
def test_rows_already_in_slot_order(device, experts, n, k, m, block_m, fuse):
    """`chord_b200_indexed_slots`: the caller has placed row s of the activations at routing
    slot s (ids are the slots themselves, padding slots hold garbage and a sentinel id).
    The rows are loaded in place; the results must be those of `indexed` /
    `indexed_gate_up_silu` on the original rows, row for row, bit for bit (same kernels,
    same tiles; only the way the rows reach shared memory differs)."""
    import chord_b200
    from chord_b200 import _lib
    from chord_b200.indexed_gemm import gemm_scratch, status_word
    from tests.cases import make_indexed_case

    case = make_indexed_case(num_experts=experts, n=n, k=k, m=m, top_k=1, block_m=block_m, seed=300 + m)
    w = chord_b200.pack_w4a16(case["codes"].to(device), case["scale"].to(device))
    sorted_ids = case["sorted_ids"].to(device)
    routing = (sorted_ids, case["expert_ids"].to(device), case["num_tokens_padded"].to(device).reshape(1))
    x = case["x"].to(device)
    width = n // 2 if fuse else n
    want = torch.full((m, width), float("nan"), dtype=torch.bfloat16, device=device)
    if fuse:
        chord_b200.indexed_gate_up_silu(x, w, *routing, 1, outputs=want, block_m=block_m)
    else:
        chord_b200.indexed(x, w, *routing, 1, outputs=want, block_m=block_m)
    # slot-ordered copy of the rows: garbage (NaN) in the padding slots
    slots = sorted_ids.numel()
    valid = sorted_ids < m
    x_slots = torch.full((slots, k), float("nan"), dtype=torch.bfloat16, device=device)
    x_slots[valid] = x[sorted_ids[valid].long()]
    slot_ids = torch.where(valid, torch.arange(slots, device=device, dtype=torch.int32),
                           torch.full_like(sorted_ids, slots))
    got = torch.full((slots, width), float("nan"), dtype=torch.bfloat16, device=device)
    lib = _lib.load()
    locks, workspace, ws_bytes = gemm_scratch(device, block_m, None, slots, k)
    _lib.check(lib.chord_b200_indexed_slots(
        x_slots.data_ptr(), w.packed.data_ptr(), w.scale.data_ptr(), slot_ids.data_ptr(), slots,
        routing[1].data_ptr(), routing[1].numel(), routing[2].data_ptr(), got.data_ptr(), 0,
        locks.data_ptr(), locks.numel(), workspace.data_ptr(), ws_bytes, status_word(device).data_ptr(),
        slots, n, k, experts, block_m, fuse, _lib.stream_handle(device)))
    torch.cuda.synchronize()
    assert int(status_word(device).item()) == 0
    # exactly the slots that hold a row are written, with the values of the original call
    assert torch.equal(~torch.isnan(got.float()).any(dim=1), valid)
    assert torch.equal(got[valid], want[sorted_ids[valid].long()])
