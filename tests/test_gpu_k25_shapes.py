"""Parity at the Kimi-K2.5 shapes the benchmark runs: the exact decode path of bench.py
(48 local of 384 experts, `indexed_block_m(..., total_experts=384)`, gate_up
4096 x 7168 and down 7168 x 2048, batches 1 / 64 / 256), `contiguous` at those shapes
with ragged row counts, and `masked` at [12, 256, 7168].

The weights are too large to dequantise in full on the CPU, so the written-row pattern
is checked for every route and the values for a sample of the reached experts, each
dequantised once (the oracle's numerics: BF16 RN((code - 8) * scale), FP32 accumulate).
The reference's own tests at these shapes: tests/test_w4a16_grouped.py:132-146, 450-469,
tests/test_w4a16_indexed.py:1262-1285.
"""

import pytest
import torch

from oracle import w4a16_oracle as O
from tests.cases import make_checkpoint_weights

pytestmark = pytest.mark.gpu

COS_INDEXED, COS_GROUPED, REL_LIMIT = 5e-3, 1e-3, 1e-2
EXPERTS_TOTAL, LOCAL, TOP_K, HIDDEN, INTER = 384, 48, 8, 7168, 2048


def expert_weight_f32(words, scale, e):
    """FP32 copy of expert e's dequantised weights, [N, K]."""
    n, k8 = words.shape[1], words.shape[2]
    codes = torch.from_numpy(O.unpack_checkpoint_uint4(words[e].numpy())).reshape(n, k8 * 8)
    return O.dequantize_bf16(codes, scale[e]).float()


def sample(items, count):
    items = list(items)
    if len(items) <= count:
        return items
    step = (len(items) - 1) / (count - 1)
    return sorted({items[round(i * step)] for i in range(count)})


@pytest.fixture(scope="module")
def k25(device):
    """The two projections' weights (48 experts each) in checkpoint form on the host and
    packed on the device, shared by the tests of this module."""
    import chord_b200

    words13, scale13 = make_checkpoint_weights(LOCAL, 2 * INTER, HIDDEN, seed=131)
    words2, scale2 = make_checkpoint_weights(LOCAL, HIDDEN, INTER, seed=132)
    w13 = chord_b200.pack_w4a16(words13.to(device), scale13.to(device), packed=True)
    w2 = chord_b200.pack_w4a16(words2.to(device), scale2.to(device), packed=True)
    return dict(words13=words13, scale13=scale13, words2=words2, scale2=scale2, w13=w13, w2=w2)


@pytest.mark.parametrize("batch", [1, 64, 256])
def test_decode_step_at_the_benchmarked_configuration(device, k25, batch):
    """gate_up -> SiLU*mul -> down exactly as bench.py's step runs them."""
    import chord_b200
    from chord_b200.indexed_gemm import status_word

    g = torch.Generator().manual_seed(9000 + batch)
    topk = O.topk_ids_random(batch, TOP_K, EXPERTS_TOTAL, g)
    if batch == 1:  # make sure the single token reaches a local expert
        topk[0, 0] = 5
    x = torch.randn((batch, HIDDEN), generator=g).to(torch.bfloat16)
    w13, w2 = k25["w13"], k25["w2"]
    block_m = chord_b200.indexed_block_m(w13, batch, TOP_K, total_experts=EXPERTS_TOTAL)
    assert block_m == 16
    routing = chord_b200.moe_align_block_size(topk.to(device), block_m, LOCAL, expert_base=0)
    routes = batch * TOP_K
    locks = torch.zeros(1024, dtype=torch.int32, device=device)
    gate_up = torch.full((routes, 2 * INTER), float("nan"), dtype=torch.bfloat16, device=device)
    hidden = torch.full((routes, INTER), float("nan"), dtype=torch.bfloat16, device=device)
    out = torch.full((routes, HIDDEN), float("nan"), dtype=torch.bfloat16, device=device)
    chord_b200.indexed(x.to(device), w13, *routing, TOP_K, locks=locks, outputs=gate_up, block_m=block_m)
    chord_b200.silu_mul(gate_up, sorted_ids=routing[0], num_tokens_padded=routing[2], outputs=hidden)
    chord_b200.indexed(hidden, w2, *routing, 1, locks=locks, outputs=out, block_m=block_m)
    # the benchmark's step takes gate_up and SiLU*mul in one launch
    fused = torch.full((routes, INTER), float("nan"), dtype=torch.bfloat16, device=device)
    chord_b200.indexed_gate_up_silu(x.to(device), w13, *routing, TOP_K, locks=locks, outputs=fused,
                                    block_m=block_m)
    torch.cuda.synchronize()
    assert int(status_word(device).item()) == 0
    assert bool((locks == 0).all())

    flat = topk.reshape(-1)
    local = flat < LOCAL
    gate_up_c, hidden_c, out_c = gate_up.float().cpu(), hidden.cpu(), out.float().cpu()
    # exactly the routes to local experts are written, in all three buffers
    for buf in (gate_up_c, hidden_c.float(), out_c):
        assert torch.equal(~torch.isnan(buf).any(dim=1), local)
        assert torch.equal(torch.isnan(buf).all(dim=1), ~local)
    reached = sorted(set(flat[local].tolist()))
    assert reached, "the draw reaches no local expert"
    for e in sample(reached, 6):
        rows = torch.where(flat == e)[0]
        tokens = torch.div(rows, TOP_K, rounding_mode="floor")
        ref13 = x[tokens].float() @ expert_weight_f32(k25["words13"], k25["scale13"], e).t()
        assert O.cosine_diff(gate_up_c[rows], ref13) <= COS_INDEXED
        assert O.max_abs_rel(gate_up_c[rows], ref13) <= REL_LIMIT
        # down on the kernel's own SiLU*mul output (the oracle's SiLU*mul is checked elsewhere)
        ref2 = hidden_c[rows].float() @ expert_weight_f32(k25["words2"], k25["scale2"], e).t()
        assert O.cosine_diff(out_c[rows], ref2) <= COS_INDEXED
        assert O.max_abs_rel(out_c[rows], ref2) <= REL_LIMIT
        # SiLU*mul on the kernel's gate_up (fast exponential on the device: one BF16 step)
        want = O.silu_mul(gate_up[rows.to(device)].cpu()).float()
        assert (hidden_c[rows].float() - want).abs().max() <= 2.0 ** -7 * want.abs().max()
        # fused launch: the activation of the FP32 gate_up result, rounded once
        act = torch.nn.functional.silu(ref13[:, :INTER]) * ref13[:, INTER:]
        fused_rows = fused[rows.to(device)].float().cpu()
        assert O.cosine_diff(fused_rows, act) <= COS_INDEXED
        assert O.max_abs_rel(fused_rows, act) <= 1.5e-2
    assert torch.equal(~torch.isnan(fused.float().cpu()).any(dim=1), local)


@pytest.mark.parametrize("projection", ["gate_up", "down"])
def test_contiguous_at_k25_shapes_with_ragged_experts(device, k25, projection):
    """Prefill layout at the K2.5 shapes: runs of 1, 127, 128 and 300 rows (padded to 128,
    256 merged tiles included), an expert without rows and a trailing padding tile."""
    import chord_b200
    from chord_b200.packing import PreparedWeight

    words, scale, w = ((k25["words13"], k25["scale13"], k25["w13"]) if projection == "gate_up"
                       else (k25["words2"], k25["scale2"], k25["w2"]))
    experts = 5
    sub = PreparedWeight(w.packed[:experts], w.scale[:experts], w.n, w.k, experts)
    counts = [1, 127, 0, 128, 300]
    idx = []
    for e, c in enumerate(counts):
        idx += [e] * c + [-1] * ((c + 127) // 128 * 128 - c)
    idx += [-1] * 128
    m_indices = torch.tensor(idx, dtype=torch.int32)
    g = torch.Generator().manual_seed(77)
    x2 = torch.randn((len(idx), w.k), generator=g).to(torch.bfloat16)
    x2[m_indices < 0] = 0
    out = torch.full((len(idx), w.n), float("nan"), dtype=torch.bfloat16, device=device)
    chord_b200.contiguous(x2.to(device), sub, m_indices.to(device), outputs=out)
    torch.cuda.synchronize()
    got = out.float().cpu()
    written = ~torch.isnan(got).any(dim=1)
    expect_written = torch.ones(len(idx), dtype=torch.bool)
    expect_written[-128:] = False          # the trailing padding tile is not touched
    assert torch.equal(written, expect_written)
    assert bool((got[(m_indices < 0) & written] == 0).all())
    for e, c in enumerate(counts):
        if c == 0:
            continue
        rows = torch.where(m_indices == e)[0]
        ref = x2[rows].float() @ expert_weight_f32(words, scale, e).t()
        assert O.cosine_diff(got[rows], ref) < COS_GROUPED
        assert O.max_abs_rel(got[rows], ref) <= REL_LIMIT


@pytest.mark.parametrize("expected_m", [8, 32, 128])
def test_masked_at_ep32_shape(device, k25, expected_m):
    """`masked` on [12, 256, 7168] (EP32) with Poisson(expected_m) row counts: rows at or
    past masked_m untouched everywhere, values checked for three groups."""
    import chord_b200
    from chord_b200.packing import PreparedWeight

    groups, max_m = 12, 256
    w = k25["w13"]
    sub = PreparedWeight(w.packed[:groups], w.scale[:groups], w.n, w.k, groups)
    g = torch.Generator().manual_seed(500 + expected_m)
    masked_m = torch.poisson(torch.full((groups,), float(expected_m)), generator=g).clamp(0, max_m)
    masked_m = masked_m.to(torch.int32)
    masked_m[3] = 0                       # an empty group
    if expected_m == 128:
        masked_m[7] = max_m               # and a full one
    x3 = torch.randn((groups, max_m, w.k), generator=g).to(torch.bfloat16)
    out = torch.full((groups * max_m, w.n), float("nan"), dtype=torch.bfloat16, device=device)
    chord_b200.masked(x3.to(device), sub, masked_m.to(device), expected_m, outputs=out)
    torch.cuda.synchronize()
    got = out.float().cpu().view(groups, max_m, w.n)
    for grp in range(groups):
        mm = int(masked_m[grp])
        assert not bool(torch.isnan(got[grp, :mm]).any())
        assert bool(torch.isnan(got[grp, mm:]).all())
    for grp in (0, 7, 11):
        mm = int(masked_m[grp])
        if mm == 0:
            continue
        ref = x3[grp, :mm].float() @ expert_weight_f32(k25["words13"], k25["scale13"], grp).t()
        assert O.cosine_diff(got[grp, :mm], ref) < COS_GROUPED
        assert O.max_abs_rel(got[grp, :mm], ref) <= REL_LIMIT
