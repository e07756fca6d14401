"""Benchmark of the W4A16 MoE expert GEMM path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--batch B]

Workload (every N): Kimi-K2.5 EP8 decode through `indexed` - 48 local experts out of
384, top_k 8, hidden 7168, expert intermediate 2048; gate_up W [48, 4096, 7168] and
down W [48, 7168, 2048] in INT4 with BF16 group-32 scales; `--batch` tokens per rank
(default 256) routed uniformly over the 384 experts, local routes kept.  One step =
gate_up -> SiLU*mul -> down on one batch.  Inputs are seeded synthetic tensors of the
benchmark's shapes and value distributions; weights are random-initialised.

With N > 1 every rank is one EP8 rank with its own batch (weak scaling, no collective
on this path), and the line also carries `ep_layer`: the full 384-expert layer
sharded over the N GPUs with NCCL all-to-all dispatch/combine (4096 tokens in total).

Prints ONE JSON line (rank 0).  `value` is microseconds per step with everything
resident in HBM; `e2e` is the same step with host buffers (pinned host -> device
copies of activations and routing, device -> host read of the result) inside the
timed region; `roofline` is algorithmic bytes of the two GEMM launches over their
CUDA-event time against the measured HBM copy bandwidth; `cpu_baseline` /
`--impl reference` time the reference's CPU torch path (oracle/w4a16_oracle.py) on a
bounded sample of the same workload.
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
FALLBACK_HBM_GBS = 6650.0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="chord_b200", choices=["chord_b200", "reference"])
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--no-ep-layer", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--all-batches", action="store_true",
                    help="also time batches 1, 16 and 64 (reported under `batches`)")
    ap.add_argument("--grouped", action="store_true",
                    help="also time the prefill (contiguous) and masked configurations "
                         "(reported under `prefill` and `masked`)")
    return ap.parse_args()


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return float(data["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


def traffic_bytes(active, n, k, in_rows, out_rows):
    """Algorithmic DRAM bytes of one GEMM launch (reference: tests/roofline.py:58-71)."""
    return active * n * (k // 2) + active * n * (k // 32) * 2 + in_rows * k * 2 + out_rows * n * 2


# ------------------------------------------------------------------- workload --

def random_prepared_weight(num_experts, n, k, device, seed, chunk=48):
    """Random checkpoint-form weights packed on the device, `chunk` experts at a time."""
    import chord_b200
    from chord_b200.packing import PreparedWeight

    g = torch.Generator(device=device).manual_seed(seed)
    packed, scales = [], []
    for start in range(0, num_experts, chunk):
        e = min(chunk, num_experts - start)
        words = torch.randint(-2**31, 2**31 - 1, (e, n, k // 8), dtype=torch.int64, device=device,
                              generator=g).to(torch.int32)
        scale = (torch.rand((e, n, k // 32), device=device, generator=g) * 0.015 + 0.005
                 ).to(torch.bfloat16)
        w = chord_b200.pack_w4a16(words, scale, packed=True)
        packed.append(w.packed)
        scales.append(w.scale)
        del words, scale
    if len(packed) == 1:
        return PreparedWeight(packed[0], scales[0], n, k, num_experts)
    return PreparedWeight(torch.cat(packed), torch.cat(scales), n, k, num_experts)


def decode_routing(batch, seed, expert_base=0):
    """Uniform top-8 of 384 per token (scores -> topk), local routes kept, aligned on CPU."""
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
        self.out_host = torch.empty((routes, HIDDEN), dtype=torch.bfloat16).pin_memory()
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

    def step_e2e(self):
        """Same step through the public API from host buffers."""
        self.x.copy_(self.x_host, non_blocking=True)
        self.sorted_ids.copy_(self.sorted_host, non_blocking=True)
        self.expert_ids.copy_(self.expert_host, non_blocking=True)
        self.padded.copy_(self.padded_host, non_blocking=True)
        self.step()
        self.out_host.copy_(self.out, non_blocking=True)

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


def time_region(step_fn, steps, warmup, world, device, min_seconds=0.0):
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


# --------------------------------------------------------------- CPU baseline --

def cpu_reference_step(batch, seed, max_experts, threads):
    """The reference's CPU torch path (BF16 dequantise, FP32 matmul; oracle port of
    tests/generators.py:259-319) for gate_up -> SiLU*mul -> down on the experts the
    batch reaches, at most `max_experts` of them.  Returns (seconds for the sample,
    experts in the sample, experts the batch reaches)."""
    from oracle import w4a16_oracle as O

    torch.set_num_threads(threads)
    topk = decode_routing(batch, seed)
    flat = topk.reshape(-1)
    active = [e for e in range(LOCAL_EXPERTS) if bool((flat == e).any())]
    sample = active[:max_experts]
    g = torch.Generator().manual_seed(seed + 1)
    x = torch.randn((batch, HIDDEN), generator=g).to(torch.bfloat16)
    wg = torch.Generator().manual_seed(7)
    elapsed = 0.0
    for e in sample:
        codes13 = torch.randint(0, 16, (2 * INTER, HIDDEN), dtype=torch.int32, generator=wg)
        scale13 = (torch.rand((2 * INTER, HIDDEN // 32), generator=wg) * 0.015 + 0.005).to(torch.bfloat16)
        codes2 = torch.randint(0, 16, (HIDDEN, INTER), dtype=torch.int32, generator=wg)
        scale2 = (torch.rand((HIDDEN, INTER // 32), generator=wg) * 0.015 + 0.005).to(torch.bfloat16)
        rows = torch.where(flat == e)[0]
        tokens = torch.div(rows, TOP_K, rounding_mode="floor")
        t0 = time.perf_counter()
        w13 = O.dequantize_bf16(codes13, scale13).float()
        gate_up = (x[tokens].float() @ w13.t()).to(torch.bfloat16)
        hidden = O.silu_mul(gate_up)
        w2 = O.dequantize_bf16(codes2, scale2).float()
        _ = (hidden.float() @ w2.t()).to(torch.bfloat16)
        elapsed += time.perf_counter() - t0
    return elapsed, len(sample), len(active)


# ------------------------------------------------------------------- EP layer --

def ep_layer_bench(device, rank, world, steps, warmup):
    """Full 384-expert layer over `world` GPUs: 4096 tokens in total, top_k 8, uniform
    routing; dispatch and combine by all_to_all_single around the local
    gate_up / SiLU*mul / down.  Strong scaling (total work fixed)."""
    from chord_b200 import ep
    from oracle import w4a16_oracle as O

    tokens_total = 4096
    local = EXPERTS_TOTAL // world
    w13 = random_prepared_weight(local, 2 * INTER, HIDDEN, device, seed=100 + rank)
    w2 = random_prepared_weight(local, HIDDEN, INTER, device, seed=200 + rank)
    g = torch.Generator().manual_seed(300)
    topk_all = O.topk_ids_random(tokens_total, TOP_K, EXPERTS_TOTAL, g)
    per_rank = tokens_total // world
    topk = topk_all[rank * per_rank:(rank + 1) * per_rank].to(device)
    xg = torch.Generator().manual_seed(400 + rank)
    x = torch.randn((per_rank, HIDDEN), generator=xg).to(torch.bfloat16).to(device)
    experts = ep.local_expert_mlp(w13, w2)
    group = torch.distributed.group.WORLD if world > 1 else None

    def step():
        return ep.moe_layer(x, topk, EXPERTS_TOTAL, experts, group=group)

    ms = time_region(step, steps, warmup, world, device)
    rows_here = int(((topk_all // local) == rank).sum())
    result = {
        "workload": "k2.5_full_layer_384_experts_4096_tokens_top8_uniform",
        "scaling": "strong", "n_gpus": world, "us_per_layer": ms * 1e3,
        "tokens_total": tokens_total, "experts_per_gpu": local, "routed_rows_rank0": rows_here,
        "collective": "none" if world == 1 else "nccl all_to_all_single (counts, dispatch, ids, combine)",
        "steps": steps, "warmup": warmup,
    }
    del w13, w2
    torch.cuda.empty_cache()
    return result


# ------------------------------------------------- prefill / masked side lines --

def _event_us(fn, reps=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) * 1e3)
    times.sort()
    return times[len(times) // 2]


def grouped_bench(device, w13, w2):
    """BASELINE configurations 3 and 4 on the weights of the decode workload.

    Prefill: 8192 tokens, top-8 by multinomial over 384 experts whose popularity is drawn
    from Dirichlet(0.5) (seeded), rows of the 48 local experts kept, grouped per expert and
    padded to 128; `contiguous` gate_up -> SiLU*mul -> `contiguous` down.  Masked: 24 local
    experts, [24, 256, K] activations, masked_m ~ Poisson(expected_m) clipped to 256."""
    import chord_b200
    from chord_b200.packing import PreparedWeight

    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    tensor_peak = float(peaks.get("bf16_tflops", 1590.0))
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
    flops = 2.0 * valid * (2 * INTER * HIDDEN + HIDDEN * INTER)
    tflops = flops / ((us_gate + us_down) * 1e-6) / 1e12
    prefill = {
        "workload": "k2.5_prefill_contiguous_8192_tokens_top8_dirichlet0.5", "rows_valid": valid,
        "rows_padded": m, "experts_reached": sum(c > 0 for c in counts),
        "gate_up_us": us_gate, "silu_mul_us": us_act, "down_us": us_down,
        "tflops_valid_rows": tflops,
        "roofline": {"bound": "tensor", "achieved": tflops, "peak": tensor_peak, "unit": "TFLOP/s",
                     "frac": tflops / tensor_peak, "peak_kind": "measured" if peaks else "fallback"},
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
        masked.append({"groups": groups, "expected_m": expected_m, "rows": rows, "gate_up_us": us1,
                       "down_us": us2, "gbs": nbytes / ((us1 + us2) * 1e-6) / 1e9,
                       "tflops": 2.0 * rows * 3 * INTER * HIDDEN / ((us1 + us2) * 1e-6) / 1e12})
    return prefill, masked


# ----------------------------------------------------------------------- main --

def run_reference_arm(args, rank, world):
    """`--impl reference`: the reference's CPU torch path on the host cores (rank 0 only)."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    max_experts = 4
    times = []
    for i in range(args.warmup + args.steps):
        seconds, sampled, active = cpu_reference_step(args.batch, seed=args.batch, max_experts=max_experts,
                                                      threads=threads)
        if i >= args.warmup:
            times.append(seconds * active / max(sampled, 1))
    value_us = sum(times) / len(times) * 1e6
    sample = (f"gate_up->SiLU*mul->down for the first {sampled} of the {active} experts the batch "
              f"reaches, per step; scaled by {active}/{sampled}")
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


def workload_config(batch):
    return {"workload": f"k2.5_ep8_decode_indexed_batch{batch}", "local_experts": LOCAL_EXPERTS,
            "experts_total": EXPERTS_TOTAL, "top_k": TOP_K, "hidden": HIDDEN, "intermediate": INTER,
            "tokens_per_rank": batch, "routing": "uniform top-8 of 384, local routes kept",
            "l2": "inputs larger than L2 (1.19 GB of weights per step vs 126 MB)"}


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
    from chord_b200 import build as native_build
    from chord_b200.indexed_gemm import status_word

    if rank == 0:
        native_build.build()
    barrier(world)

    w13 = random_prepared_weight(LOCAL_EXPERTS, 2 * INTER, HIDDEN, device, seed=1 + rank)
    w2 = random_prepared_weight(LOCAL_EXPERTS, HIDDEN, INTER, device, seed=2 + rank)
    workload = DecodeWorkload(device, args.batch, seed=args.batch + 1000 * rank, w13=w13, w2=w2)

    with ClockSampler(local_rank) as sampler:
        ms = time_region(workload.step, args.steps, args.warmup, world, device)
        kernel_us = time_kernels(workload, max(args.steps, 5))
        e2e_ms = time_region(lambda: (workload.step_e2e(), torch.cuda.synchronize()), args.steps,
                             args.warmup, world, device)
    clocks = sampler.summary()
    assert int(status_word(device).item()) == 0, "a kernel gave up on a bounded wait"

    batches = {}
    if args.all_batches:
        for b in (1, 16, 64):
            wl = DecodeWorkload(device, b, seed=b + 1000 * rank, w13=w13, w2=w2)
            t = time_region(wl.step, args.steps, args.warmup, world, device)
            k_us = time_kernels(wl, max(args.steps, 5))
            gemm_bytes = wl.bytes_gate_up + wl.bytes_down
            graph_us = None
            try:
                # the same step replayed from a CUDA graph (what a decode loop would do)
                side = torch.cuda.Stream(device)
                side.wait_stream(torch.cuda.current_stream(device))
                with torch.cuda.stream(side):
                    wl.step()
                torch.cuda.current_stream(device).wait_stream(side)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    wl.step()
                graph_us = time_region(graph.replay, args.steps, args.warmup, world, device) * 1e3
            except Exception:  # noqa: BLE001 - the eager number above stands on its own
                graph_us = None
            batches[str(b)] = {"us": t * 1e3, "graph_replay_us": graph_us, "gate_up_us": k_us[0], "silu_mul_us": k_us[1],
                               "down_us": k_us[2], "active_experts": wl.active, "routed_rows": wl.routed,
                               "block_m": wl.block_m,
                               "gemm_gbs": gemm_bytes / ((k_us[0] + k_us[2]) * 1e-6) / 1e9 if wl.active else None}

    prefill = masked = None
    if args.grouped:
        prefill, masked = grouped_bench(device, w13, w2)

    ep_layer = None
    if not args.no_ep_layer:
        ep_layer = ep_layer_bench(device, rank, world, max(3, min(args.steps, 5)), 3)

    peak, peak_kind = measured_peaks()
    gemm_bytes = workload.bytes_gate_up + workload.bytes_down
    gemm_us = kernel_us[0] + kernel_us[2]
    achieved = gemm_bytes / (gemm_us * 1e-6) / 1e9 if gemm_us > 0 else 0.0
    cpu = None
    if rank == 0 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        seconds, sampled, active = cpu_reference_step(args.batch, seed=args.batch, max_experts=4,
                                                      threads=threads)
        cpu = {"value": seconds * active / max(sampled, 1) * 1e6, "unit": "us", "cores": threads,
               "kind": "port",
               "sample": f"gate_up->SiLU*mul->down for {sampled} of {active} reached experts, "
                         f"scaled by {active}/{sampled}"}
    if rank == 0:
        line = {
            "metric": METRIC, "value": ms * 1e3, "unit": "us", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(args.batch),
            "kernels_us": {"gate_up": kernel_us[0], "silu_mul": kernel_us[1], "down": kernel_us[2]},
            "routing": {"block_m": workload.block_m, "active_experts": workload.active,
                        "routed_rows": workload.routed},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_kind": peak_kind,
                         "kernel": ("w4a16_decode_kernel" if workload.block_m <= 32
                                    else "w4a16_gemm_kernel") + " (gate_up + down launches)",
                         "algorithmic_bytes_per_step": gemm_bytes,
                         # dram__bytes_read+write of one ncu capture of both launches at batch
                         # 256 (1208.0 MB for 48 reached experts), scaled by the experts this
                         # step reaches
                         "traffic": 1208.0e6 * workload.active / 48.0,
                         "traffic_source": "profiles/w4a16_decode_kernel_k25_ep8_decode.md"},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_ms * 1e3, "unit": "us", "h2d_bytes_per_step": workload.h2d_bytes,
                    "d2h_bytes_per_step": workload.d2h_bytes},
            "gpu_launches": 3 * args.steps * world,
            "clocks": clocks,
        }
        if batches:
            line["batches"] = batches
        if prefill is not None:
            line["prefill"], line["masked"] = prefill, masked
        if ep_layer is not None:
            line["ep_layer"] = ep_layer
        print(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
