"""Benchmark of the W4A16 MoE expert GEMM path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--batch B]

Headline workload (every N): Kimi-K2.5 EP8 decode through `indexed` - 48 local experts
out of 384, top_k 8, hidden 7168, expert intermediate 2048; gate_up W [48, 4096, 7168]
and down W [48, 7168, 2048] in INT4 with BF16 group-32 scales; `--batch` tokens per rank
(default 256) routed uniformly over the 384 experts, local routes kept.  One step =
gate_up -> SiLU*mul -> down on one batch.  Inputs are seeded synthetic tensors of the
benchmark's shapes and value distributions; weights are random-initialised.

With N > 1 every rank is one EP8 rank with its own batch (weak scaling, no collective on
this path).  The same line carries, measured in the same run:
  parity     the benchmarked step's outputs against the CPU oracle on sampled experts,
             computed before anything is timed
  batches    the step at 1 / 16 / 64 tokens per rank (eager and CUDA-graph replay)
  prefill    `contiguous` on 8192 tokens with Dirichlet(0.5) expert popularity (tensor roofline)
  masked     `masked` on [24, 256, K] with Poisson row counts
  ep_layer   the full 384-expert layer sharded over the N GPUs, 4096 tokens in total,
             tokens exchanged by the library's kernels over peer memory (strong scaling),
             with its own parity check and the time of the same layer on NCCL all-to-all
  reference_gpu   (only when CHORD_REFERENCE names a checkout of the reference that is
             importable on this machine) the reference's own `indexed` kernel on the same
             inputs, at its own block size and at block_m 8 and 16

Prints ONE JSON line (rank 0).  `value` is microseconds per step with everything resident
in HBM; `e2e` is the same step with host buffers (pinned host -> device copies of
activations and routing, device -> host read of the result: the output rows of the routes
to local experts, gathered on the device; the other rows of the [routes, N] buffer are
never written) inside the timed region;
`roofline` is algorithmic bytes of the two GEMM launches over their CUDA-event time
against the measured HBM copy bandwidth; `cpu_baseline` / `--impl reference` time the
reference's CPU torch path (oracle/w4a16_oracle.py) on a bounded sample of the workload.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

EXPERTS_TOTAL, LOCAL_EXPERTS, TOP_K, HIDDEN, INTER = 384, 48, 8, 7168, 2048
METRIC = "gate_up+down_us"
FALLBACK_HBM_GBS, FALLBACK_TFLOPS = 6650.0, 1590.0
COS_LIMIT, REL_LIMIT = 5e-3, 1e-2          # per GEMM: the reference's limit and BASELINE's
CHAIN_REL_LIMIT = 2e-2                     # gate_up -> SiLU*mul -> down checked end to end


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="chord_b200", choices=["chord_b200", "reference"])
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--no-ep-layer", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-side-lines", action="store_true",
                    help="skip batches / prefill / masked / sustained (short runs under a profiler)")
    ap.add_argument("--no-parity", action="store_true")
    return ap.parse_args()


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]),
                "bf16_tflops_sustained": float(data.get("bf16_tflops_sustained", data["bf16_tflops"])),
                "kind": "measured"}
    return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_TFLOPS,
            "bf16_tflops_sustained": 1400.0, "kind": "fallback"}


def recorded_traffic():
    """DRAM bytes per step of the decode kernel's two launches from the committed ncu
    capture (profiles/w4a16_decode_kernel_traffic.json), or None."""
    path = ROOT / "profiles" / "w4a16_decode_kernel_traffic.json"
    if not path.exists():
        return None
    return json.loads(path.read_text())


def traffic_bytes(active, n, k, in_rows, out_rows):
    """Algorithmic DRAM bytes of one GEMM launch (reference: tests/roofline.py:58-71)."""
    return active * n * (k // 2) + active * n * (k // 32) * 2 + in_rows * k * 2 + out_rows * n * 2


# ------------------------------------------------------------------- workload --

def random_prepared_weight(num_experts, n, k, device, seed, chunk=48, keep=()):
    """Random checkpoint-form weights packed on the device, `chunk` experts at a time.
    Returns the PreparedWeight and, for the experts in `keep`, their checkpoint words and
    scales on the host (for the parity checks)."""
    import chord_b200
    from chord_b200.packing import PreparedWeight

    g = torch.Generator(device=device).manual_seed(seed)
    packed, scales, kept = [], [], {}
    for start in range(0, num_experts, chunk):
        e = min(chunk, num_experts - start)
        words = torch.randint(-2**31, 2**31 - 1, (e, n, k // 8), dtype=torch.int64, device=device,
                              generator=g).to(torch.int32)
        scale = (torch.rand((e, n, k // 32), device=device, generator=g) * 0.015 + 0.005
                 ).to(torch.bfloat16)
        for idx in keep:
            if start <= idx < start + e:
                kept[idx] = (words[idx - start].cpu(), scale[idx - start].cpu())
        w = chord_b200.pack_w4a16(words, scale, packed=True)
        packed.append(w.packed)
        scales.append(w.scale)
        del words, scale
    if len(packed) == 1:
        return PreparedWeight(packed[0], scales[0], n, k, num_experts), kept
    return PreparedWeight(torch.cat(packed), torch.cat(scales), n, k, num_experts), kept


def dequantized_f32(words, scale):
    """FP32 copy of one expert's weights from checkpoint words [N, K/8] and scales [N, K/32]
    with the oracle's numerics (BF16 RN((code - 8) * scale))."""
    from oracle import w4a16_oracle as O

    n, k8 = words.shape
    codes = torch.from_numpy(O.unpack_checkpoint_uint4(words.numpy())).reshape(n, k8 * 8)
    return O.dequantize_bf16(codes, scale).float()


def decode_routing(batch, seed):
    """Uniform top-8 of 384 per token (scores -> topk), as tests/generators.py:174-189."""
    from oracle import w4a16_oracle as O

    g = torch.Generator().manual_seed(seed)
    return O.topk_ids_random(batch, TOP_K, EXPERTS_TOTAL, g)


class DecodeWorkload:
    def __init__(self, device, batch, seed, w13, w2):
        import chord_b200
        from chord_b200 import fused_ops

        self.device, self.batch, self.w13, self.w2 = device, batch, w13, w2
        self.topk = decode_routing(batch, seed)
        self.block_m = chord_b200.indexed_block_m(w13, batch, TOP_K, total_experts=EXPERTS_TOTAL)
        topk_dev = self.topk.to(device)
        self.sorted_ids, self.expert_ids, self.padded = fused_ops.moe_align_block_size(
            topk_dev, self.block_m, LOCAL_EXPERTS, expert_base=0)
        count = int(self.padded.item())
        self.routed = int((self.sorted_ids[:count] < batch * TOP_K).sum().item()) if count else 0
        self.active = int(torch.unique(self.expert_ids[: count // self.block_m]).numel()) if count else 0
        g = torch.Generator().manual_seed(seed + 1)
        self.x_host = torch.randn((batch, HIDDEN), generator=g).to(torch.bfloat16).pin_memory()
        self.x = self.x_host.to(device)
        routes = batch * TOP_K
        self.gate_up = torch.empty((routes, 2 * INTER), dtype=torch.bfloat16, device=device)
        self.hidden = torch.empty((routes, INTER), dtype=torch.bfloat16, device=device)
        self.out = torch.empty((routes, HIDDEN), dtype=torch.bfloat16, device=device)
        self.locks = torch.zeros(1024, dtype=torch.int32, device=device)
        # host copies for the end-to-end arm
        self.sorted_host = self.sorted_ids.cpu().pin_memory()
        self.expert_host = self.expert_ids.cpu().pin_memory()
        self.padded_host = self.padded.cpu().pin_memory()
        # The step's result is the rows of the routes to local experts (the only rows of
        # `out` the kernels write): they are gathered on the device and read back compactly.
        flat = self.topk.reshape(-1)
        self.local_routes = torch.nonzero(flat < LOCAL_EXPERTS).reshape(-1).to(device)
        self.out_local = torch.empty((self.local_routes.numel(), HIDDEN), dtype=torch.bfloat16, device=device)
        self.out_host = torch.empty((self.local_routes.numel(), HIDDEN), dtype=torch.bfloat16).pin_memory()
        self.bytes_gate_up = traffic_bytes(self.active, 2 * INTER, HIDDEN, batch, self.routed)
        self.bytes_down = traffic_bytes(self.active, HIDDEN, INTER, self.routed, self.routed)

    def step(self, events=None):
        import chord_b200

        routing = (self.sorted_ids, self.expert_ids, self.padded)
        if events:
            events[0].record()
        chord_b200.indexed(self.x, self.w13, *routing, TOP_K, locks=self.locks,
                           outputs=self.gate_up, block_m=self.block_m)
        if events:
            events[1].record()
        chord_b200.silu_mul(self.gate_up, sorted_ids=self.sorted_ids, num_tokens_padded=self.padded,
                            outputs=self.hidden)
        if events:
            events[2].record()
        chord_b200.indexed(self.hidden, self.w2, *routing, 1, locks=self.locks, outputs=self.out,
                           block_m=self.block_m)
        if events:
            events[3].record()

    def step_fused(self):
        """The same step with SiLU*mul in gate_up's epilogue (two launches).  Measured
        beside `step`: at these tile sizes it is the slower of the two."""
        import chord_b200

        routing = (self.sorted_ids, self.expert_ids, self.padded)
        chord_b200.indexed_gate_up_silu(self.x, self.w13, *routing, TOP_K, locks=self.locks,
                                        outputs=self.hidden, block_m=self.block_m)
        chord_b200.indexed(self.hidden, self.w2, *routing, 1, locks=self.locks, outputs=self.out,
                           block_m=self.block_m)

    def step_e2e(self):
        """Same step through the public API from host buffers."""
        self.x.copy_(self.x_host, non_blocking=True)
        self.sorted_ids.copy_(self.sorted_host, non_blocking=True)
        self.expert_ids.copy_(self.expert_host, non_blocking=True)
        self.padded.copy_(self.padded_host, non_blocking=True)
        self.step()
        torch.index_select(self.out, 0, self.local_routes, out=self.out_local)
        self.out_host.copy_(self.out_local, non_blocking=True)

    @property
    def h2d_bytes(self):
        return (self.x_host.numel() * 2 + self.sorted_host.numel() * 4 + self.expert_host.numel() * 4
                + 4)

    @property
    def d2h_bytes(self):
        return self.out_host.numel() * 2


# --------------------------------------------------------------------- timing --

class ClockSampler:
    """Samples SM clock and throttle reasons (read-only NVML queries) in a background
    thread while the timed region runs."""

    def __init__(self, index):
        self.index, self.samples, self.reasons, self.max_mhz = index, [], 0, None
        self.stop = threading.Event()
        self.thread = None

    def __enter__(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            index = self.index
            if visible:
                entry = visible.split(",")[self.index].strip()
                index = int(entry) if entry.isdigit() else self.index
            handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))

            def poll():
                while not self.stop.is_set():
                    try:
                        self.samples.append(int(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)))
                        self.reasons |= int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle))
                    except Exception:
                        break
                    time.sleep(0.001)

            self.thread = threading.Thread(target=poll, daemon=True)
            self.thread.start()
        except Exception:
            self.thread = None
        return self

    def __exit__(self, *exc):
        self.stop.set()
        if self.thread is not None:
            self.thread.join(timeout=2)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        bits = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20,
                "hw_thermal_slowdown": 0x40}
        clocks = sorted(self.samples)
        return {"sm_mhz": clocks[len(clocks) // 2], "sm_max_mhz": self.max_mhz,
                "reasons": [name for name, bit in bits.items() if self.reasons & bit],
                "samples": len(clocks)}


def barrier(world):
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()


def max_over_ranks(value, world, device):
    if world == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return float(t.item())


def time_region(step_fn, steps, warmup, world, device):
    """W untimed steps, then exactly K steps between barrier + synchronize, timed with
    CUDA events on the launching stream; returns ms per step (max over ranks)."""
    for _ in range(warmup):
        step_fn()
    barrier(world)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        step_fn()
    stop.record()
    barrier(world)
    return max_over_ranks(start.elapsed_time(stop) / steps, world, device)


def time_sustained(step_fn, seconds, probe_ms, local_rank):
    """The same step back to back for about `seconds`, with the SM clock sampled over
    that stretch: the decode kernel is bound by instruction issue, so its time follows
    the clock, which settles below the burst clock under sustained load."""
    steps = max(20, int(seconds * 1e3 / max(probe_ms, 1e-3)))
    with ClockSampler(local_rank) as sampler:
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            step_fn()
        stop.record()
        torch.cuda.synchronize()
    clocks = sampler.summary()
    us = start.elapsed_time(stop) / steps * 1e3
    ratio = (clocks["sm_mhz"] / clocks["sm_max_mhz"]) if clocks["sm_mhz"] and clocks["sm_max_mhz"] else None
    return {"seconds": start.elapsed_time(stop) / 1e3, "steps": steps, "us_per_step": us,
            "sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"],
            "us_scaled_to_max_clock": us * ratio if ratio else None}


def time_kernels(workload, steps):
    """Per-kernel CUDA-event durations (us) of gate_up, SiLU*mul and down, averaged."""
    sums = [0.0, 0.0, 0.0]
    sets = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(steps)]
    for ev in sets:
        workload.step(ev)
    torch.cuda.synchronize()
    for ev in sets:
        for i in range(3):
            sums[i] += ev[i].elapsed_time(ev[i + 1]) * 1e3
    return [s / steps for s in sums]


def _event_us(fn, reps=10, warmup=3, flush=None):
    """Median CUDA-event time of one call, optionally with L2 flushed before each."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(reps):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) * 1e3)
    times.sort()
    return times[len(times) // 2]


# --------------------------------------------------------------------- parity --

def _metrics(got, ref):
    from oracle import w4a16_oracle as O

    return O.cosine_diff(got, ref), O.max_abs_rel(got, ref)


def decode_parity(workload, kept13, kept2):
    """The benchmarked step's outputs against the CPU oracle on the experts in `kept13`
    (checkpoint words and scales kept on the host): gate_up from the activations, down
    from the kernel's own SiLU*mul output, the fused gate_up + SiLU*mul launch against
    silu(gate) * up of the oracle's FP32 result; and exactly the local routes are written."""
    nan = float("nan")
    for buf in (workload.gate_up, workload.hidden, workload.out):
        buf.fill_(nan)
    workload.step()
    torch.cuda.synchronize()
    flat = workload.topk.reshape(-1)
    local = flat < LOCAL_EXPERTS
    gate_up, hidden, out = workload.gate_up.float().cpu(), workload.hidden.cpu(), workload.out.float().cpu()
    rows_ok = all(torch.equal(~torch.isnan(buf).any(dim=1), local) for buf in (gate_up, hidden.float(), out))
    workload.hidden.fill_(nan)
    workload.step_fused()
    torch.cuda.synchronize()
    fused = workload.hidden.float().cpu()
    rows_ok = rows_ok and torch.equal(~torch.isnan(fused).any(dim=1), local)
    worst = {"gate_up": [0.0, 0.0], "down": [0.0, 0.0], "gate_up_silu_fused": [0.0, 0.0]}
    x = workload.x_host
    for e in sorted(kept13):
        rows = torch.where(flat == e)[0]
        if rows.numel() == 0:
            continue
        tokens = torch.div(rows, TOP_K, rounding_mode="floor")
        ref13 = x[tokens].float() @ dequantized_f32(*kept13[e]).t()
        act = torch.nn.functional.silu(ref13[:, :INTER]) * ref13[:, INTER:]
        for name, got, ref in (
            ("gate_up", gate_up[rows], ref13),
            ("down", out[rows], hidden[rows].float() @ dequantized_f32(*kept2[e]).t()),
            ("gate_up_silu_fused", fused[rows], act),
        ):
            cos, rel = _metrics(got, ref)
            worst[name] = [max(worst[name][0], cos), max(worst[name][1], rel)]
    ok = rows_ok and all(worst[n][0] <= COS_LIMIT and worst[n][1] <= REL_LIMIT for n in ("gate_up", "down"))
    ok = ok and worst["gate_up_silu_fused"][0] <= COS_LIMIT and worst["gate_up_silu_fused"][1] <= CHAIN_REL_LIMIT
    result = {"checked_experts": sorted(kept13), "rows_written_match_routing": bool(rows_ok)}
    for name, (cos, rel) in worst.items():
        result[name] = {"cos_diff": cos, "max_abs_rel": rel}
    result["limits"] = {"cos_diff": COS_LIMIT, "max_abs_rel": REL_LIMIT,
                        "max_abs_rel_after_activation": CHAIN_REL_LIMIT}
    result["ok"] = bool(ok)
    return result


# --------------------------------------------------------------- CPU baseline --

_CPU_WEIGHTS = None


def cpu_reference_step(batch, seed, threads):
    """The reference's CPU torch path (BF16 dequantise, FP32 matmul; oracle port of
    tests/generators.py:259-319) for gate_up -> SiLU*mul -> down on every expert the batch
    reaches, each with its own rows.  Two experts' worth of random codes and scales are
    generated once and used in turn (the values do not change the work; at 117 MB per
    matrix nothing stays in cache between experts).  Returns (seconds, experts reached)."""
    from oracle import w4a16_oracle as O

    global _CPU_WEIGHTS
    torch.set_num_threads(threads)
    if _CPU_WEIGHTS is None:
        wg = torch.Generator().manual_seed(7)
        _CPU_WEIGHTS = []
        for _ in range(2):
            codes13 = torch.randint(0, 16, (2 * INTER, HIDDEN), dtype=torch.int32, generator=wg)
            scale13 = (torch.rand((2 * INTER, HIDDEN // 32), generator=wg) * 0.015 + 0.005).to(torch.bfloat16)
            codes2 = torch.randint(0, 16, (HIDDEN, INTER), dtype=torch.int32, generator=wg)
            scale2 = (torch.rand((HIDDEN, INTER // 32), generator=wg) * 0.015 + 0.005).to(torch.bfloat16)
            _CPU_WEIGHTS.append((codes13, scale13, codes2, scale2))
    topk = decode_routing(batch, seed)
    flat = topk.reshape(-1)
    active = [e for e in range(LOCAL_EXPERTS) if bool((flat == e).any())]
    g = torch.Generator().manual_seed(seed + 1)
    x = torch.randn((batch, HIDDEN), generator=g).to(torch.bfloat16)
    elapsed = 0.0
    for i, e in enumerate(active):
        codes13, scale13, codes2, scale2 = _CPU_WEIGHTS[i % 2]
        rows = torch.where(flat == e)[0]
        tokens = torch.div(rows, TOP_K, rounding_mode="floor")
        t0 = time.perf_counter()
        w13 = O.dequantize_bf16(codes13, scale13).float()
        gate_up = (x[tokens].float() @ w13.t()).to(torch.bfloat16)
        hidden = O.silu_mul(gate_up)
        w2 = O.dequantize_bf16(codes2, scale2).float()
        _ = (hidden.float() @ w2.t()).to(torch.bfloat16)
        elapsed += time.perf_counter() - t0
    return elapsed, len(active)


# ------------------------------------------------------------------- EP layer --

def ep_layer_bench(device, rank, world, steps, warmup, check_parity):
    """Full 384-expert layer over `world` GPUs: 4096 tokens in total, top_k 8, uniform
    routing; tokens exchanged by the library's kernels over peer memory around the local
    gate_up / SiLU*mul / down (strong scaling: total work fixed).  Also times the same
    layer with NCCL all_to_all_single for comparison, and checks a sample of this rank's
    returned routes against the CPU oracle."""
    from chord_b200 import ep
    from oracle import w4a16_oracle as O

    tokens_total = 4096
    local = EXPERTS_TOTAL // world
    w13, kept13 = random_prepared_weight(local, 2 * INTER, HIDDEN, device, seed=100 + rank, keep=(0,))
    w2, kept2 = random_prepared_weight(local, HIDDEN, INTER, device, seed=200 + rank, keep=(0,))
    g = torch.Generator().manual_seed(300)
    topk_all = O.topk_ids_random(tokens_total, TOP_K, EXPERTS_TOTAL, g)
    per_rank = tokens_total // world
    topk_host = topk_all[rank * per_rank:(rank + 1) * per_rank].contiguous()
    topk = topk_host.to(device)
    xg = torch.Generator().manual_seed(400 + rank)
    x_host = torch.randn((per_rank, HIDDEN), generator=xg).to(torch.bfloat16)
    x = x_host.to(device)
    group = torch.distributed.group.WORLD if world > 1 else None
    layer = ep.ExpertParallelLayer(w13, w2, num_experts_total=EXPERTS_TOTAL, max_tokens=per_rank,
                                   top_k=TOP_K, group=group)

    parity = None
    if check_parity:
        out = layer(x, topk).float().cpu().reshape(per_rank * TOP_K, HIDDEN)
        # expert 0 of this rank and of the next one: a local route and one that crossed NVLink
        owners = sorted({rank, (rank + 1) % world})
        if world > 1:
            gathered = []
            for words, scale in (kept13[0], kept2[0]):
                for t in (words, scale):
                    mine = t.to(device)
                    parts = [torch.empty_like(mine) for _ in range(world)]
                    torch.distributed.all_gather(parts, mine)
                    gathered.append([p.cpu() for p in parts])
            w13_words, w13_scale, w2_words, w2_scale = gathered
        else:
            w13_words, w13_scale = [kept13[0][0]], [kept13[0][1]]
            w2_words, w2_scale = [kept2[0][0]], [kept2[0][1]]
        flat = topk_host.reshape(-1)
        cos_worst = rel_worst = 0.0
        checked = 0
        for owner in owners:
            rows = torch.where(flat == owner * local)[0]
            if rows.numel() == 0:
                continue
            tokens = torch.div(rows, TOP_K, rounding_mode="floor")
            d13 = dequantized_f32(w13_words[owner], w13_scale[owner])
            d2 = dequantized_f32(w2_words[owner], w2_scale[owner])
            gate_up = (x_host[tokens].float() @ d13.t()).to(torch.bfloat16)
            ref = O.silu_mul(gate_up).float() @ d2.t()
            cos, rel = _metrics(out[rows], ref)
            cos_worst, rel_worst, checked = max(cos_worst, cos), max(rel_worst, rel), checked + rows.numel()
        status = layer.status()
        verdict = torch.tensor([cos_worst, rel_worst, float(status), float(torch.isnan(out).any())],
                               dtype=torch.float64, device=device)
        if world > 1:
            torch.distributed.all_reduce(verdict, op=torch.distributed.ReduceOp.MAX)
        cos_worst, rel_worst, status, has_nan = (float(v) for v in verdict.cpu())
        parity = {"routes_checked_rank0": checked, "owners_checked_per_rank": len(owners),
                  "cos_diff": cos_worst, "max_abs_rel": rel_worst, "exchange_status": int(status),
                  "limits": {"cos_diff": COS_LIMIT, "max_abs_rel": CHAIN_REL_LIMIT},
                  "ok": bool(cos_worst <= COS_LIMIT and rel_worst <= CHAIN_REL_LIMIT and status == 0
                             and has_nan == 0)}

    ms = time_region(lambda: layer(x, topk), steps, warmup, world, device)
    # where the time goes: CUDA events around the steps of three more calls
    layer.spans = []
    for _ in range(3):
        layer(x, topk)
    torch.cuda.synchronize()
    spans = {}
    for name, start, stop in layer.spans:
        spans[name] = spans.get(name, 0.0) + start.elapsed_time(stop) * 1e3 / 3
    layer.spans = None
    spans = {k: max_over_ranks(v, world, device) for k, v in sorted(spans.items())}

    nccl_us = None
    if world > 1:
        experts = ep.local_expert_mlp(w13, w2)
        nccl_ms = time_region(lambda: ep.moe_layer(x, topk, EXPERTS_TOTAL, experts, group=group),
                              max(3, steps // 2), 2, world, device)
        nccl_us = nccl_ms * 1e3
    rows_here = int(((topk_all // local) == rank).sum())
    flops = 2.0 * rows_here * 3 * INTER * HIDDEN
    result = {
        "workload": "k2.5_full_layer_384_experts_4096_tokens_top8_uniform",
        "scaling": "strong", "n_gpus": world, "us_per_layer": ms * 1e3,
        "tokens_total": tokens_total, "experts_per_gpu": local, "routed_rows_rank0": rows_here,
        "exchange": "none" if world == 1 else
                    "own kernels over peer memory: dispatch by peer stores, combine by the down "
                    "projection's epilogue storing into the source rank's result tensor",
        "spans_us": spans,
        "gemm_us": spans.get("experts"),
        "comm_us": None if world == 1 else sum(v for k, v in spans.items() if k != "experts"),
        "tflops_rank0": flops / (ms * 1e-3) / 1e12,
        "nccl_all_to_all_us": nccl_us, "parity": parity, "steps": steps, "warmup": warmup,
    }
    del w13, w2, layer
    torch.cuda.empty_cache()
    return result


# ------------------------------------------------- prefill / masked side lines --

def grouped_bench(device, w13, w2, peaks):
    """BASELINE configurations 3 and 4 on the weights of the decode workload.

    Prefill: 8192 tokens, top-8 by multinomial over 384 experts whose popularity is drawn
    from Dirichlet(0.5) (seeded), rows of the 48 local experts kept, grouped per expert and
    padded to 128; `contiguous` gate_up -> SiLU*mul -> `contiguous` down.  Masked: 24 local
    experts, [24, 256, K] activations, masked_m ~ Poisson(expected_m) clipped to 256."""
    import chord_b200
    from chord_b200.packing import PreparedWeight

    tensor_peak = peaks["bf16_tflops"]
    g = torch.Generator().manual_seed(3)
    torch.manual_seed(3)
    popularity = torch.distributions.Dirichlet(torch.full((EXPERTS_TOTAL,), 0.5)).sample()
    topk = torch.multinomial(popularity.expand(8192, EXPERTS_TOTAL), TOP_K, replacement=False, generator=g)
    counts = [int((topk == e).sum()) for e in range(LOCAL_EXPERTS)]
    idx = []
    for e, c in enumerate(counts):
        idx += [e] * c + [-1] * ((c + 127) // 128 * 128 - c)
    m_indices = torch.tensor(idx, dtype=torch.int32, device=device)
    m, valid = m_indices.numel(), sum(counts)
    x = torch.randn((m, HIDDEN), device=device).to(torch.bfloat16)
    x[m_indices < 0] = 0
    gate_up = torch.empty((m, 2 * INTER), dtype=torch.bfloat16, device=device)
    hidden = torch.empty((m, INTER), dtype=torch.bfloat16, device=device)
    out = torch.empty((m, HIDDEN), dtype=torch.bfloat16, device=device)
    us_gate = _event_us(lambda: chord_b200.contiguous(x, w13, m_indices, outputs=gate_up))
    us_act = _event_us(lambda: chord_b200.silu_mul(gate_up, outputs=hidden))
    us_down = _event_us(lambda: chord_b200.contiguous(hidden, w2, m_indices, outputs=out))
    active = sum(c > 0 for c in counts)
    flops = 2.0 * valid * (2 * INTER * HIDDEN + HIDDEN * INTER)
    nbytes = (traffic_bytes(active, 2 * INTER, HIDDEN, valid, valid)
              + traffic_bytes(active, HIDDEN, INTER, valid, valid))
    gemm_s = (us_gate + us_down) * 1e-6
    tflops = flops / gemm_s / 1e12
    # the slower of FLOPs at the tensor peak and bytes at the HBM peak bounds the two GEMMs
    floor_us = max(flops / (tensor_peak * 1e12), nbytes / (peaks["hbm_gbs"] * 1e9)) * 1e6
    prefill = {
        "workload": "k2.5_prefill_contiguous_8192_tokens_top8_dirichlet0.5", "rows_valid": valid,
        "rows_padded": m, "experts_reached": active,
        "experts_below_128_rows": sum(0 < c < 128 for c in counts),
        "gate_up_us": us_gate, "silu_mul_us": us_act, "down_us": us_down,
        "tflops_valid_rows": tflops, "gbs": nbytes / gemm_s / 1e9,
        "roofline": {"bound": "tensor", "achieved": tflops, "peak": tensor_peak, "unit": "TFLOP/s",
                     "frac": tflops / tensor_peak, "peak_kind": peaks["kind"],
                     "frac_of_sustained_peak": tflops / peaks["bf16_tflops_sustained"],
                     "roofline_us": floor_us, "frac_of_roofline_time": floor_us / (us_gate + us_down),
                     "traffic": None},
    }
    masked = []
    groups = 24
    wa = PreparedWeight(w13.packed[:groups], w13.scale[:groups], w13.n, w13.k, groups)
    wb = PreparedWeight(w2.packed[:groups], w2.scale[:groups], w2.n, w2.k, groups)
    for expected_m in (8, 32, 128):
        gm = torch.Generator().manual_seed(expected_m)
        masked_m = torch.poisson(torch.full((groups,), float(expected_m)), generator=gm).clamp(0, 256)
        masked_m = masked_m.to(torch.int32)
        rows, active = int(masked_m.sum()), int((masked_m > 0).sum())
        mm = masked_m.to(device)
        x3 = torch.randn((groups, 256, HIDDEN), device=device).to(torch.bfloat16)
        h3 = torch.randn((groups, 256, INTER), device=device).to(torch.bfloat16)
        o1 = torch.empty((groups * 256, 2 * INTER), dtype=torch.bfloat16, device=device)
        o2 = torch.empty((groups * 256, HIDDEN), dtype=torch.bfloat16, device=device)
        us1 = _event_us(lambda: chord_b200.masked(x3, wa, mm, expected_m, outputs=o1))
        us2 = _event_us(lambda: chord_b200.masked(h3, wb, mm, expected_m, outputs=o2))
        nbytes = traffic_bytes(active, 2 * INTER, HIDDEN, rows, rows) + traffic_bytes(active, HIDDEN, INTER, rows, rows)
        flops = 2.0 * rows * 3 * INTER * HIDDEN
        floor_us = max(flops / (tensor_peak * 1e12), nbytes / (peaks["hbm_gbs"] * 1e9)) * 1e6
        masked.append({"groups": groups, "expected_m": expected_m, "rows": rows, "gate_up_us": us1,
                       "down_us": us2, "gbs": nbytes / ((us1 + us2) * 1e-6) / 1e9,
                       "tflops": flops / ((us1 + us2) * 1e-6) / 1e12,
                       "roofline_us": floor_us, "frac_of_roofline_time": floor_us / (us1 + us2)})
    return prefill, masked


# ------------------------------------- the reference's own GPU kernel (optional) --

def reference_gpu_bench(device, w13, w2):
    """When CHORD_REFERENCE names a checkout of the reference that imports here, time its
    `indexed` (its Blackwell mma.sync schedule, compiled by its own NVRTC pipeline) on the
    decode inputs of this benchmark: at its own `indexed_block_m` and with block_m 8 and 16
    passed through its public override (chord_kernels/ops.py:8-19); this library's kernel is
    timed the same way beside it (L2 flushed before every call, median of 10)."""
    root = os.environ.get("CHORD_REFERENCE")
    if not root or not (Path(root) / "chord_kernels").is_dir():
        return None
    import tempfile

    from oracle import w4a16_oracle as O

    scratch = tempfile.mkdtemp(prefix="chord_ref_")
    os.environ.setdefault("CHORD_TMP_DIR", os.path.join(scratch, "tmp"))
    os.environ.setdefault("CHORD_CACHE_DIR", os.path.join(scratch, "cache"))
    sys.path.insert(0, root)
    try:
        import chord_b200
        import chord_kernels as ref
        from chord_kernels.operator.packing import PreparedWeight as RefWeight
    except Exception as exc:  # noqa: BLE001
        return {"unavailable": f"{type(exc).__name__}: {exc}"}
    if Path(getattr(ref, "__file__", "")).resolve().parent == ROOT / "chord_kernels":
        return {"unavailable": "CHORD_REFERENCE resolves to this repository's own chord_kernels shim"}
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.int8, device=device)
    rows_out = []
    try:
        for batch in (16, 64, 256):
            topk = decode_routing(batch, batch)
            g = torch.Generator().manual_seed(batch + 1)
            for name, ours in (("gate_up", w13), ("down", w2)):
                theirs = RefWeight(ours.packed, ours.scale, ours.n, ours.k, ours.num_experts)  # same bytes
                rows = batch if name == "gate_up" else batch * TOP_K
                x = torch.randn((rows, ours.k), generator=g).to(torch.bfloat16).to(device)
                outp = torch.empty((batch * TOP_K, ours.n), dtype=torch.bfloat16, device=device)
                locks = torch.zeros(1024, dtype=torch.int32, device=device)
                tk = TOP_K if name == "gate_up" else 1
                entry = {"batch": batch, "projection": name}
                own_bm = int(ref.indexed_block_m(theirs, batch, TOP_K))
                for label, block_m in (("own", own_bm), ("bm8", 8), ("bm16", 16)):
                    s, e, p = O.align_routing_blocks(topk, block_m, LOCAL_EXPERTS, 0)
                    sd, ed, pd = s.to(device), e.to(device), p.to(device).reshape(1)
                    us = _event_us(lambda: ref.indexed(x, theirs, sd, ed, pd, tk, locks=locks, outputs=outp,
                                                       block_m=block_m), flush=flush)
                    entry[f"reference_{label}_us"] = us
                    if label == "own":
                        entry["reference_own_block_m"] = own_bm
                        active = int(torch.unique(e).numel())
                        routed = int((s < batch * TOP_K).sum())
                        entry["bytes"] = traffic_bytes(active, ours.n, ours.k, rows, routed)
                bm = chord_b200.indexed_block_m(ours, batch, TOP_K, total_experts=EXPERTS_TOTAL)
                s, e, p = O.align_routing_blocks(topk, bm, LOCAL_EXPERTS, 0)
                sd, ed, pd = s.to(device), e.to(device), p.to(device).reshape(1)
                entry["chord_b200_us"] = _event_us(
                    lambda: chord_b200.indexed(x, ours, sd, ed, pd, tk, locks=locks, outputs=outp, block_m=bm),
                    flush=flush)
                entry["chord_b200_block_m"] = bm
                best = min(entry[f"reference_{label}_us"] for label in ("own", "bm8", "bm16"))
                entry["reference_best_us"] = best
                entry["speedup_vs_reference_best"] = best / entry["chord_b200_us"]
                entry["chord_b200_gbs"] = entry["bytes"] / entry["chord_b200_us"] / 1e3
                entry["reference_best_gbs"] = entry["bytes"] / best / 1e3
                rows_out.append(entry)
    except Exception as exc:  # noqa: BLE001
        return {"unavailable": f"{type(exc).__name__}: {exc}", "rows": rows_out}
    return {"kernel": "reference `indexed` (NVRTC, mma.sync) on this GPU, same packed weights and routing draw",
            "timing": "CUDA events, L2 flushed before each call, median of 10", "rows": rows_out}


# ----------------------------------------------------------------------- main --

def workload_config(batch, pdl=None):
    cfg = {"workload": f"k2.5_ep8_decode_indexed_batch{batch}", "local_experts": LOCAL_EXPERTS,
           "experts_total": EXPERTS_TOTAL, "top_k": TOP_K, "hidden": HIDDEN, "intermediate": INTER,
           "tokens_per_rank": batch, "routing": "uniform top-8 of 384, local routes kept",
           "l2": "inputs larger than L2 (1.19 GB of weights per step vs 126 MB)"}
    if pdl is not None:
        cfg["programmatic_dependent_launch"] = bool(pdl)
    return cfg


def run_reference_arm(args, rank, world):
    """`--impl reference`: the reference's CPU torch path on the host cores (rank 0 only)."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    times = []
    for i in range(args.warmup + args.steps):
        seconds, active = cpu_reference_step(args.batch, seed=args.batch, threads=threads)
        if i >= args.warmup:
            times.append(seconds)
    value_us = sum(times) / len(times) * 1e6
    sample = (f"gate_up->SiLU*mul->down on all {active} experts the batch reaches, every step "
              "(dequantise each expert once in BF16, FP32 matmul on its rows)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value_us, "unit": "us", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": value_us / 1e3,
        "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": workload_config(args.batch),
        "cpu_baseline": {"value": value_us, "unit": "us", "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value_us, "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def graph_replay_us(workload, steps, warmup, world, device):
    """The step replayed from a CUDA graph (what a decode loop would do), or None."""
    try:
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            workload.step()
        torch.cuda.current_stream(device).wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            workload.step()
        return time_region(graph.replay, steps, warmup, world, device) * 1e3
    except Exception:  # noqa: BLE001 - the eager number stands on its own
        return None


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: chord_b200 has no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.distributed.init_process_group("nccl", device_id=device)
    import chord_b200
    from chord_b200 import build as native_build

    if rank == 0:
        native_build.build()
    barrier(world)
    pdl = os.environ.get("CHORD_B200_PDL", "1") != "0"
    chord_b200.set_option("pdl", 1 if pdl else 0)
    peaks = measured_peaks()

    # the experts whose weights stay on the host for the parity check: three the batch reaches
    flat = decode_routing(args.batch, args.batch + 1000 * rank).reshape(-1)
    reached = sorted(set(flat[flat < LOCAL_EXPERTS].tolist()))
    keep = tuple(sorted({reached[0], reached[len(reached) // 2], reached[-1]})) if reached else ()
    if args.no_parity:
        keep = ()
    w13, kept13 = random_prepared_weight(LOCAL_EXPERTS, 2 * INTER, HIDDEN, device, seed=1 + rank, keep=keep)
    w2, kept2 = random_prepared_weight(LOCAL_EXPERTS, HIDDEN, INTER, device, seed=2 + rank, keep=keep)
    workload = DecodeWorkload(device, args.batch, seed=args.batch + 1000 * rank, w13=w13, w2=w2)

    parity = None
    if keep:
        parity = decode_parity(workload, kept13, kept2)
        chord_b200.check_status(device)
        verdict = torch.tensor([0.0 if parity["ok"] else 1.0], dtype=torch.float64, device=device)
        if world > 1:
            torch.distributed.all_reduce(verdict, op=torch.distributed.ReduceOp.MAX)
        parity["ok_on_every_rank"] = bool(verdict.item() == 0)

    with ClockSampler(local_rank) as sampler:
        ms = time_region(workload.step, args.steps, args.warmup, world, device)
        kernel_us = time_kernels(workload, max(args.steps, 5))
        fused_us = time_region(workload.step_fused, args.steps, args.warmup, world, device) * 1e3
        e2e_ms = time_region(lambda: (workload.step_e2e(), torch.cuda.synchronize()), args.steps,
                             args.warmup, world, device)
    clocks = sampler.summary()
    chord_b200.check_status(device)

    sustained = batches = prefill = masked = None
    if not args.no_side_lines:
        sustained = time_sustained(workload.step, 1.0, ms, local_rank)
        batches = {}
        for b in (1, 16, 64):
            wl = DecodeWorkload(device, b, seed=b + 1000 * rank, w13=w13, w2=w2)
            t = time_region(wl.step, args.steps, args.warmup, world, device)
            k_us = time_kernels(wl, max(args.steps, 5))
            gemm_bytes = wl.bytes_gate_up + wl.bytes_down
            batches[str(b)] = {
                "us": t * 1e3, "graph_replay_us": graph_replay_us(wl, args.steps, args.warmup, world, device),
                "gate_up_us": k_us[0], "silu_mul_us": k_us[1], "down_us": k_us[2],
                "active_experts": wl.active, "routed_rows": wl.routed, "block_m": wl.block_m,
                "gemm_gbs": gemm_bytes / ((k_us[0] + k_us[2]) * 1e-6) / 1e9 if wl.active else None}
        if rank == 0:
            prefill, masked = grouped_bench(device, w13, w2, peaks)
        barrier(world)
    reference_gpu = reference_gpu_bench(device, w13, w2) if rank == 0 else None
    barrier(world)
    chord_b200.check_status(device)

    facts = {"block_m": workload.block_m, "active_experts": workload.active, "routed_rows": workload.routed,
             "h2d": workload.h2d_bytes, "d2h": workload.d2h_bytes,
             "gemm_bytes": workload.bytes_gate_up + workload.bytes_down}
    ep_layer = None
    if not args.no_ep_layer:
        del workload
        ep_layer = ep_layer_bench(device, rank, world, max(3, min(args.steps, 10)), 3,
                                  check_parity=not args.no_parity)

    cpu = None
    if rank == 0 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        seconds, active = cpu_reference_step(args.batch, seed=args.batch, threads=threads)
        cpu = {"value": seconds * 1e6, "unit": "us", "cores": threads, "kind": "port",
               "sample": f"one step: gate_up->SiLU*mul->down on all {active} reached experts"}
    if rank == 0:
        gemm_us = kernel_us[0] + kernel_us[2]
        achieved = facts["gemm_bytes"] / (gemm_us * 1e-6) / 1e9 if gemm_us > 0 else 0.0
        recorded = recorded_traffic()
        traffic = None
        if recorded is not None:
            # captured with every local expert reached; scaled by the experts this step reaches
            traffic = recorded["dram_bytes_per_step"] * facts["active_experts"] / recorded["active_experts"]
        line = {
            "metric": METRIC, "value": ms * 1e3, "unit": "us", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(args.batch, pdl),
            "kernels_us": {"gate_up": kernel_us[0], "silu_mul": kernel_us[1], "down": kernel_us[2]},
            "fused_gate_up_silu_step_us": fused_us,
            "routing": {k: facts[k] for k in ("block_m", "active_experts", "routed_rows")},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "peak_kind": peaks["kind"],
                         "frac_of_nominal_8tbs": achieved / 8000.0,
                         "kernel": ("w4a16_decode_kernel" if facts["block_m"] <= 32
                                    else "w4a16_gemm_kernel") + " (gate_up + down launches)",
                         "algorithmic_bytes_per_step": facts["gemm_bytes"],
                         "traffic": traffic,
                         "traffic_source": None if recorded is None else
                         f"profiles/w4a16_decode_kernel_traffic.json (kernel at commit {recorded['kernel_commit']})"},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_ms * 1e3, "unit": "us", "h2d_bytes_per_step": facts["h2d"],
                    "d2h_bytes_per_step": facts["d2h"]},
            "gpu_launches": 3 * args.steps * world,
            "clocks": clocks,
        }
        for key, value in (("parity", parity), ("sustained", sustained), ("batches", batches),
                           ("prefill", prefill), ("masked", masked), ("ep_layer", ep_layer),
                           ("reference_gpu", reference_gpu)):
            if value is not None:
                line[key] = value
        print(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
