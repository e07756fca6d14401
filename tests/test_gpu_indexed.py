"""`indexed` on the GPU against the CPU oracle (same seeded inputs), through the C ABI.

Tolerances: cosine difference <= 5e-3 (tests/test_w4a16_indexed.py:63 of the reference)
and max-abs error / max-abs reference <= 1e-2 (BF16 output with FP32 accumulation)."""

import pytest
import torch

from oracle import w4a16_oracle as O
from tests.cases import make_checkpoint_weights, make_indexed_case

pytestmark = pytest.mark.gpu

COS_LIMIT = 5e-3
REL_LIMIT = 1e-2


def run_case(device, case, *, locks=None, outputs=None, prefill=float("nan")):
    import chord_b200
    from chord_b200.indexed_gemm import status_word

    weight = chord_b200.pack_w4a16(case["codes"].to(device), case["scale"].to(device))
    m = case["topk_ids"].size(0)
    routes = m * case["top_k"]
    sorted_ids, expert_ids = case["sorted_ids"], case["expert_ids"]
    if sorted_ids.numel() == 0:          # nothing routed here: buffers may be over-allocated
        sorted_ids = torch.zeros(case["block_m"], dtype=torch.int32)
        expert_ids = torch.zeros(1, dtype=torch.int32)
    if outputs is None:
        outputs = torch.full((routes, weight.n), prefill, dtype=torch.bfloat16, device=device)
    if locks is None:
        locks = torch.zeros(1024, dtype=torch.int32, device=device)
    kernel_top_k = 1 if case["projection"] == "down" else case["top_k"]
    out = chord_b200.indexed(case["x"].to(device), weight, sorted_ids.to(device), expert_ids.to(device),
                             case["num_tokens_padded"].to(device).reshape(1), kernel_top_k,
                             locks=locks, outputs=outputs, block_m=case["block_m"])
    torch.cuda.synchronize()
    assert int(status_word(device).item()) == 0, "a kernel gave up on a bounded wait"
    assert bool((locks == 0).all()), "locks must be left zeroed"
    return out, weight


def check_against_oracle(out, case):
    ref = O.reference_indexed(case["x"], case["codes"], case["scale"], case["topk_ids"], case["top_k"],
                              projection=case["projection"], expert_base=case["expert_base"])
    got = out.float().cpu()
    written = ~torch.isnan(got).any(dim=1)
    expected = ~torch.isnan(ref).any(dim=1)
    assert torch.equal(written, expected), "rows written differ from the rows routed to local experts"
    assert not torch.isnan(got[written]).any()
    if expected.any():
        assert O.cosine_diff(got[expected], ref[expected]) <= COS_LIMIT
        assert O.max_abs_rel(got[expected], ref[expected]) <= REL_LIMIT


CASES = {
    # BASELINE config 1: E=8, K=512, N=1024, 64 tokens, top_k=2
    "config1": dict(num_experts=8, n=1024, k=512, m=64, top_k=2, block_m=16, seed=3),
    "config1_down": dict(num_experts=8, n=1024, k=512, m=64, top_k=2, block_m=16, seed=4,
                         projection="down"),
    # the reference's tiny GPU case 8x128x128, E=4
    "tiny": dict(num_experts=4, n=128, k=128, m=8, top_k=1, block_m=8, seed=11),
    "block8": dict(num_experts=8, n=1024, k=512, m=64, top_k=2, block_m=8, seed=12),
    "block24_odd_shapes": dict(num_experts=6, n=19 * 128, k=64 * 37, m=40, top_k=3, block_m=24, seed=18),
    "block64": dict(num_experts=8, n=1024, k=512, m=64, top_k=2, block_m=64, seed=13),
    "block128": dict(num_experts=4, n=256, k=2048, m=300, top_k=4, block_m=128, seed=14),
    "block256": dict(num_experts=2, n=256, k=1024, m=700, top_k=2, block_m=256, seed=15),
    "ep_window": dict(num_experts=12, n=256, k=512, m=50, top_k=4, block_m=16, seed=16,
                      experts_total=96, expert_base=24),
    "single_token": dict(num_experts=8, n=256, k=256, m=1, top_k=2, block_m=16, seed=17),
    "k64": dict(num_experts=3, n=128, k=64, m=9, top_k=2, block_m=16, seed=19),
}


@pytest.mark.parametrize("name", list(CASES))
def test_indexed_matches_oracle(device, name):
    case = make_indexed_case(**CASES[name])
    out, _ = run_case(device, case)
    check_against_oracle(out, case)


OPTION_DEFAULTS = {"dequant_groups": 2, "decode_kernel": 1, "ksplit": 1, "pregather": 1}


def _with_options(device, case, options):
    from chord_b200 import _lib

    for name, value in options.items():
        _lib.set_option(name, value)
    try:
        out, _ = run_case(device, case)
    finally:
        for name in options:
            _lib.set_option(name, OPTION_DEFAULTS.get(name, 0))
    return out


@pytest.mark.parametrize("option,value", [("x_load", 1), ("dequant_groups", 4), ("issuers", 1),
                                          ("max_stages", 2), ("grid_limit", 5)])
def test_kernel_variants_agree_bit_for_bit(device, option, value):
    """General kernel (the decode-sized one switched off): gather by TMA gather4 instead
    of cp.async, four dequant groups, one issuer, a shallow pipeline, a five-CTA grid:
    the schedule changes, the numbers must not (except the accumulation split, which
    stays within tolerance)."""
    case = make_indexed_case(num_experts=8, n=1024, k=512, m=64, top_k=2, block_m=16, seed=3)
    base = _with_options(device, case, {"decode_kernel": 0})
    out = _with_options(device, case, {"decode_kernel": 0, option: value})
    check_against_oracle(base, case)
    check_against_oracle(out, case)
    if option in ("x_load", "max_stages"):
        assert torch.equal(out.view(torch.int16), base.view(torch.int16))


@pytest.mark.parametrize("name", ["config1", "tiny", "block8", "block24_odd_shapes"])
@pytest.mark.parametrize("option,value", [("max_stages", 4), ("grid_limit", 5), ("decode_kernel", 0)])
def test_decode_kernel_variants(device, name, option, value):
    """Token tiles of at most 32 rows run on the decode-sized kernel by default; a shallow
    ring and a five-CTA grid (every tile through stream-K) must not change a bit, and the
    general kernel must agree within tolerance."""
    case = make_indexed_case(**CASES[name])
    base, _ = run_case(device, case)
    out = _with_options(device, case, {option: value})
    check_against_oracle(base, case)
    check_against_oracle(out, case)
    if option == "max_stages":
        assert torch.equal(out.view(torch.int16), base.view(torch.int16))


@pytest.mark.parametrize("name", ["block64", "block128", "block256"])
def test_routed_rows_copied_or_gathered_in_kernel(device, name):
    """Blocks of 64+ rows: the slot-ordered copy of the routed rows (default) and the
    in-kernel gather (the path a caller with the small workspace gets) both match the
    oracle; so does the copy path without the second MMA issuer."""
    case = make_indexed_case(**CASES[name])
    copied, _ = run_case(device, case)
    check_against_oracle(copied, case)
    check_against_oracle(_with_options(device, case, {"pregather": 0}), case)
    check_against_oracle(_with_options(device, case, {"ksplit": 0}), case)


def test_golden_fixture(device):
    """Inputs and FP32 reference produced by the reference's own generators."""
    from pathlib import Path

    import numpy as np

    import chord_b200

    z = np.load(Path(__file__).resolve().parent / "golden" / "mid.npz")
    e, n, k, m, top_k, block_m = (int(v) for v in z["shape"])
    bf = lambda a: torch.from_numpy(a.copy()).view(torch.bfloat16)
    weight = chord_b200.pack_w4a16(torch.from_numpy(z["checkpoint"]).to(device),
                                   bf(z["scale"]).to(device), packed=True)
    locks = torch.zeros(1024, dtype=torch.int32, device=device)
    args = (torch.from_numpy(z["sorted_ids"]).to(device), torch.from_numpy(z["expert_ids"]).to(device),
            torch.tensor([int(z["num_tokens_padded"])], dtype=torch.int32, device=device))
    gate_up = chord_b200.indexed(bf(z["x"]).to(device), weight, *args, top_k, locks=locks, block_m=block_m)
    down = chord_b200.indexed(bf(z["x_routed"]).to(device), weight, *args, 1, locks=locks, block_m=block_m)
    for got, key in ((gate_up, "ref_gate_up"), (down, "ref_down")):
        ref = torch.from_numpy(z[key].copy()).view(torch.float32)
        assert O.cosine_diff(got.float().cpu(), ref) <= COS_LIMIT
        assert O.max_abs_rel(got.float().cpu(), ref) <= REL_LIMIT


def test_deterministic_and_locks_reused(device):
    """Five launches on one lock buffer: bit-equal outputs, locks left zero
    (reference: tests/test_w4a16_indexed.py:1262-1285, 1384-1437)."""
    case = make_indexed_case(num_experts=8, n=1024, k=2048, m=24, top_k=2, block_m=16, seed=21)
    locks = torch.zeros(1024, dtype=torch.int32, device=device)
    outs = [run_case(device, case, locks=locks)[0].clone() for _ in range(5)]
    for other in outs[1:]:
        assert torch.equal(other.view(torch.int16), outs[0].view(torch.int16))
    check_against_oracle(outs[0], case)


@pytest.mark.parametrize("groups,decode_kernel", [(2, 0), (4, 0), (2, 1)])
def test_repeatable_with_every_group_count(device, groups, decode_kernel):
    """Ten launches, stream-K on every tile: bit-equal every time, on the general kernel
    with 2 and 4 dequant groups (which also changes the number of MMA issuers and the
    depth of the operand ring; guards the rule that ring depths are multiples of the
    parties taking turns on them) and on the decode-sized kernel."""
    from chord_b200 import _lib

    case = make_indexed_case(num_experts=6, n=512, k=7168, m=12, top_k=2, block_m=16, seed=26)
    _lib.set_option("dequant_groups", groups)
    _lib.set_option("decode_kernel", decode_kernel)
    try:
        outs = [run_case(device, case)[0].clone() for _ in range(10)]
    finally:
        _lib.set_option("dequant_groups", 2)
        _lib.set_option("decode_kernel", 1)
    check_against_oracle(outs[0], case)
    for other in outs[1:]:
        assert torch.equal(other.view(torch.int16), outs[0].view(torch.int16))


@pytest.mark.parametrize("decode_kernel", [1, 0])
def test_stream_k_split_matches_whole_tiles(device, decode_kernel):
    """Few tiles on many CTAs forces every tile through the stream-K reduction; a
    one-CTA grid computes whole tiles.  FP32 partials summed once: nearly all outputs
    are bit-equal; the bound is the reference's 99.5 % (tests/test_w4a16_indexed.py:1284-1285)."""
    from chord_b200 import _lib

    case = make_indexed_case(num_experts=2, n=256, k=7168, m=6, top_k=1, block_m=16, seed=22)
    _lib.set_option("decode_kernel", decode_kernel)
    try:
        split, _ = run_case(device, case)
        _lib.set_option("grid_limit", 1)
        whole, _ = run_case(device, case)
    finally:
        _lib.set_option("grid_limit", 0)
        _lib.set_option("decode_kernel", 1)
    check_against_oracle(split, case)
    check_against_oracle(whole, case)
    a, b = split.float().cpu(), whole.float().cpu()
    rows = ~torch.isnan(a).any(dim=1)
    same = float((a[rows] == b[rows]).float().mean())
    assert same >= 0.995, f"only {same:.4f} of the outputs are bit-equal"
    assert O.max_abs_rel(a[rows], b[rows]) < 1e-2


def test_empty_routing_and_untouched_rows(device):
    """num_tokens_padded == 0 launches and exits; rows no id names keep their contents."""
    case = make_indexed_case(num_experts=4, n=256, k=256, m=5, top_k=2, block_m=16, seed=23,
                             experts_total=400, expert_base=300)
    case["topk_ids"] = case["topk_ids"].clamp(max=250)       # nothing lands in [300, 304)
    case["sorted_ids"], case["expert_ids"], case["num_tokens_padded"] = O.align_routing_blocks(
        case["topk_ids"], 16, 4, 300)
    assert int(case["num_tokens_padded"]) == 0
    out, _ = run_case(device, case, prefill=3.0)
    assert bool((out == 3.0).all())
    # over-allocated routing buffers: entries past num_tokens_padded are never read
    case = make_indexed_case(num_experts=8, n=256, k=256, m=20, top_k=2, block_m=16, seed=24)
    case["sorted_ids"] = torch.cat([case["sorted_ids"], torch.full((64,), -12345, dtype=torch.int32)])
    case["expert_ids"] = torch.cat([case["expert_ids"], torch.full((4,), 999, dtype=torch.int32)])
    out, _ = run_case(device, case)
    check_against_oracle(out, case)


def test_full_size_decode_shape_properties(device):
    """K2.5 EP8 gate_up shape (48 local of 384 experts, top_k 8), 16 tokens per rank.
    Too large for the CPU oracle in full, so: (1) oracle on the routed rows only (the
    oracle touches only the experts that were reached), (2) linearity in x."""
    import chord_b200

    e, n, k, m, top_k = 48, 4096, 7168, 16, 8
    words, scale = make_checkpoint_weights(e, n, k, seed=31)
    weight = chord_b200.pack_w4a16(words.to(device), scale.to(device), packed=True)
    g = torch.Generator().manual_seed(32)
    x = torch.randn((m, k), generator=g).to(torch.bfloat16)
    topk = O.topk_ids_random(m, top_k, 384, g)
    block_m = chord_b200.indexed_block_m(weight, m, top_k)
    sorted_ids, expert_ids, padded = O.align_routing_blocks(topk, block_m, e, 0)
    locks = torch.zeros(1024, dtype=torch.int32, device=device)
    args = (weight, sorted_ids.to(device), expert_ids.to(device), padded.to(device).reshape(1), top_k)
    out = torch.full((m * top_k, n), float("nan"), dtype=torch.bfloat16, device=device)
    chord_b200.indexed(x.to(device), *args, locks=locks, outputs=out, block_m=block_m)
    codes = torch.from_numpy(O.unpack_checkpoint_uint4(words.numpy())).reshape(e, n, k)
    ref = O.reference_indexed(x, codes, scale, topk, top_k)
    got = out.float().cpu()
    rows = ~torch.isnan(ref).any(dim=1)
    assert torch.equal(rows, ~torch.isnan(got).any(dim=1))
    assert O.cosine_diff(got[rows], ref[rows]) <= COS_LIMIT
    assert O.max_abs_rel(got[rows], ref[rows]) <= REL_LIMIT
    # linearity: doubling x doubles every output exactly (power-of-two scaling is exact in BF16)
    out2 = torch.full_like(out, float("nan"))
    chord_b200.indexed((x * 2).to(device), *args, locks=locks, outputs=out2, block_m=block_m)
    assert torch.equal((out2.float().cpu()[rows]), got[rows] * 2)


def test_argument_checks(device):
    import chord_b200

    case = make_indexed_case(num_experts=4, n=128, k=128, m=8, top_k=1, block_m=8, seed=11)
    w = chord_b200.pack_w4a16(case["codes"].to(device), case["scale"].to(device))
    x = case["x"].to(device)
    s, e = case["sorted_ids"].to(device), case["expert_ids"].to(device)
    p = case["num_tokens_padded"].to(device).reshape(1)
    with pytest.raises(ValueError, match="top_k"):
        chord_b200.indexed(x, w, s, e, p, 0)
    with pytest.raises(TypeError):
        chord_b200.indexed(x, w, s.long(), e, p, 1)
    with pytest.raises(ValueError, match="multiple of 8"):
        chord_b200.indexed(x, w, s, e, p, 1, block_m=12)
    with pytest.raises(ValueError, match="does not match"):
        chord_b200.indexed(x[:, :64].contiguous(), w, s, e, p, 1)
    with pytest.raises(RuntimeError, match="lock words"):
        chord_b200.indexed(x, w, s, e, p, 1, locks=torch.zeros(4, dtype=torch.int32, device=device))
    with pytest.raises(ValueError, match="prefix"):
        bad = torch.full_like(s, 8)      # sentinel everywhere ...
        bad[1] = 0                       # ... then a routed id after a sentinel
        chord_b200.indexed(x, w, bad, e, p, 1, block_m=8, validate_routing=True)
    out = chord_b200.indexed(x, w, s, e, p, 1, block_m=8, validate_routing=True)  # locks=None is fine
    assert out.shape == (8, 128)


def test_decode_step_replays_from_a_cuda_graph(device):
    """gate_up -> SiLU*mul -> down captured once and replayed: the launches allocate only
    from torch's (graph-pool aware) caching allocator and never synchronise, so a decode
    loop can run them from a CUDA graph (reference: tests/test_w4a16_indexed.py:1208-1259).
    Replays on new activations must match eager launches bit for bit."""
    import chord_b200
    from chord_b200.indexed_gemm import status_word

    case = make_indexed_case(num_experts=8, n=1024, k=512, m=64, top_k=2, block_m=16, seed=41)
    codes2, scale2 = make_checkpoint_weights(8, 512, 512, seed=42)
    w13 = chord_b200.pack_w4a16(case["codes"].to(device), case["scale"].to(device))
    w2 = chord_b200.pack_w4a16(codes2.to(device), scale2.to(device), packed=True)
    routing = (case["sorted_ids"].to(device), case["expert_ids"].to(device),
               case["num_tokens_padded"].to(device).reshape(1))
    locks = torch.zeros(1024, dtype=torch.int32, device=device)
    x = case["x"].to(device).clone()
    gate_up = torch.zeros((128, 1024), dtype=torch.bfloat16, device=device)
    hidden = torch.zeros((128, 512), dtype=torch.bfloat16, device=device)
    out = torch.zeros((128, 512), dtype=torch.bfloat16, device=device)

    def step():
        chord_b200.indexed(x, w13, *routing, 2, locks=locks, outputs=gate_up, block_m=16)
        chord_b200.silu_mul(gate_up, sorted_ids=routing[0], num_tokens_padded=routing[2], outputs=hidden)
        chord_b200.indexed(hidden, w2, *routing, 1, locks=locks, outputs=out, block_m=16)

    side = torch.cuda.Stream(device)
    side.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(side):
        for _ in range(2):
            step()
    torch.cuda.current_stream(device).wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    g = torch.Generator().manual_seed(43)
    for _ in range(3):
        x.copy_(torch.randn(x.shape, generator=g).to(torch.bfloat16))
        graph.replay()
        torch.cuda.synchronize()
        replayed = out.clone()
        step()
        torch.cuda.synchronize()
        assert torch.equal(replayed.view(torch.int16), out.view(torch.int16))
    assert int(status_word(device).item()) == 0
    assert bool((locks == 0).all())


def test_lock_wait_gives_up_and_reports(device):
    """The bounded wait of a stream-K owner, made to run out without hanging anything: the
    lock words start at a large negative value, so the contributors' increments never
    reach the count the owner waits for.  With the poll limit set low the launch returns
    at once, the status word carries the lock-timeout bit, check_status() raises, and a
    following launch on zeroed locks is correct again."""
    import chord_b200
    from chord_b200 import _lib
    from chord_b200.indexed_gemm import status_word

    case = make_indexed_case(num_experts=2, n=256, k=7168, m=6, top_k=1, block_m=16, seed=22)
    weight = chord_b200.pack_w4a16(case["codes"].to(device), case["scale"].to(device))
    args = (case["x"].to(device), weight, case["sorted_ids"].to(device), case["expert_ids"].to(device),
            case["num_tokens_padded"].to(device).reshape(1), 1)
    poisoned = torch.full((1024,), -(1 << 20), dtype=torch.int32, device=device)
    out = torch.zeros((6, 256), dtype=torch.bfloat16, device=device)
    _lib.set_option("lock_spins", 64)
    try:
        chord_b200.indexed(*args, locks=poisoned, outputs=out, block_m=16)
        torch.cuda.synchronize()
    finally:
        _lib.set_option("lock_spins", 1 << 22)
    assert int(status_word(device).item()) & 16, "the owner's lock wait should have run out"
    with pytest.raises(RuntimeError, match="lock"):
        chord_b200.check_status(device)
    assert int(status_word(device).item()) == 0      # check_status clears the word
    good, _ = run_case(device, case)                  # fresh locks: correct again
    check_against_oracle(good, case)


def test_programmatic_dependent_launch_gives_the_same_bits(device):
    """gate_up -> SiLU*mul -> down with option pdl = 1 (each launch may become resident
    while its predecessor drains and synchronises with it through griddepcontrol.wait;
    the reference sets the same launch attribute for enable_pdl,
    csrc/launcher/launcher.cpp:440-451): bit-equal to the plain launches, repeatedly."""
    import chord_b200
    from chord_b200 import _lib

    case = make_indexed_case(num_experts=8, n=1024, k=512, m=64, top_k=2, block_m=16, seed=51)
    codes2, scale2 = make_checkpoint_weights(8, 512, 512, seed=52)
    w13 = chord_b200.pack_w4a16(case["codes"].to(device), case["scale"].to(device))
    w2 = chord_b200.pack_w4a16(codes2.to(device), scale2.to(device), packed=True)
    routing = (case["sorted_ids"].to(device), case["expert_ids"].to(device),
               case["num_tokens_padded"].to(device).reshape(1))
    locks = torch.zeros(1024, dtype=torch.int32, device=device)
    x = case["x"].to(device)

    def step():
        gate_up = chord_b200.indexed(x, w13, *routing, 2, locks=locks, block_m=16)
        hidden = chord_b200.silu_mul(gate_up, sorted_ids=routing[0], num_tokens_padded=routing[2])
        return chord_b200.indexed(hidden, w2, *routing, 1, locks=locks, block_m=16)

    plain = step().clone()
    _lib.set_option("pdl", 1)
    try:
        for _ in range(5):
            assert torch.equal(step().view(torch.int16), plain.view(torch.int16))
    finally:
        _lib.set_option("pdl", 0)
    chord_b200.check_status(device)
    assert bool((locks == 0).all())
