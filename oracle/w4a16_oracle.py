"""CPU restatement of the reference's W4A16 MoE GEMM path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product (``chord_b200/``) may import this module: it is the
checker used by ``tests/``, by ``__graft_entry__.smoke()`` and by the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``.

Every function follows one piece of the reference (novitalabs/chord,
``chord_kernels``) and cites it.  Parity pinning: the functions here are
checked, in ``tests/test_oracle.py``, against golden vectors produced by
running the reference's own CPU-runnable code (``tests/generators.py`` and
``chord_kernels/operator/packing.py::_pack_weight_scale``) - see
``tests/golden/make_golden.py``.  The packed-weight layout has no golden vector
or known-answer test in the reference (its only producer is a CUDA kernel):
``repack_literal`` restates that kernel thread by thread, ``repack_closed_form`` is
checked against it, and both are checked bit for bit against the words the
reference's own ``pack_w4a16`` produced on a B200
(``tests/golden/reference_gpu.npz``, made by
``tests/golden/make_reference_gpu_golden.py``); ``reference_indexed`` is checked
against the BF16 output of the reference's ``indexed`` kernel from the same run.
``reference_masked`` / ``reference_contiguous`` are checked against the inputs and
expected outputs the reference's own grouped tests build on the CPU
(``make_masked_case`` / ``make_contiguous_case``, ``tests/golden/grouped.npz``).
"""

from __future__ import annotations

import math

import numpy as np
import torch

GROUP = 32  # K elements per scale


# --------------------------------------------------------------------- packing --

def pack_checkpoint_uint4(codes: np.ndarray) -> np.ndarray:
    """Eight little-endian 4-bit codes per int32 word.

    Follows tests/generators.py:322-327 (``pack_checkpoint_uint4``).
    """
    codes = np.asarray(codes).astype(np.uint64)
    words = codes.reshape(*codes.shape[:-1], -1, 8)
    shifts = (np.arange(8, dtype=np.uint64) * 4)
    packed = (words << shifts).sum(axis=-1).astype(np.uint64)
    return (packed & 0xFFFFFFFF).astype(np.uint32).view(np.int32)


def unpack_checkpoint_uint4(words: np.ndarray) -> np.ndarray:
    """Inverse of :func:`pack_checkpoint_uint4` (``load_uint4<true>``,
    include/humming/kernel/repack.cuh:36-42)."""
    w = np.asarray(words).view(np.uint32).astype(np.uint64)
    shifts = (np.arange(8, dtype=np.uint64) * 4)
    nibbles = (w[..., None] >> shifts) & 0xF
    return nibbles.reshape(*w.shape[:-1], -1).astype(np.int32)


def _pack_fragment_literal(values: np.ndarray, interleave_mode: int) -> np.ndarray:
    """``pack_w4a16_fragment`` (repack.cuh:8-33) for one lane: 128 codes -> 16 words."""
    out = np.zeros(16, dtype=np.uint64)

    def interleaved_index(index: int) -> int:
        return (index % 4) * 2 + index // 4

    for i in range(4):
        for bit in range(4):
            packed = 0
            for k in range(8):
                permuted = interleaved_index(k)
                low_source = k if interleave_mode % 2 == 0 else permuted
                high_source = k if interleave_mode // 2 == 0 else permuted
                base = i * 32 + bit * 8
                packed |= (int(values[base + low_source]) & 0x7) << (k * 4)
                packed |= (int(values[base + high_source]) & 0x8) << (k * 4)
            out[i * 4 + bit] = packed
    return out


def repack_literal(codes: np.ndarray) -> np.ndarray:
    """Thread-by-thread emulation of ``repack_w4a16`` (repack.cuh:48-121) as the
    reference launches it: grid (ceil(N/64), ceil(K/64), E), 32 lanes, interleave
    mode 3 (chord_kernels/operator/kernel/repack_weight.py:41-77).

    ``codes`` int [E, N, K] in [0, 15] -> int32 [E, K/16, 2N].  Slow (pure Python
    loops): for small shapes only.
    """
    codes = np.asarray(codes)
    e_count, n, k = codes.shape
    assert n % 64 == 0 and k % 64 == 0
    out = np.zeros((e_count * (k // 16), 2 * n), dtype=np.uint64)
    for e in range(e_count):
        for bx in range(n // 64):
            for by in range(k // 64):
                smem = codes[e, bx * 64:(bx + 1) * 64, by * 64:(by + 1) * 64]
                for lane in range(32):
                    # fragment[4][1][4][2][2][2] flattened
                    fragment = np.zeros((4, 1, 4, 2, 2, 2), dtype=np.int64)
                    for i in range(8):
                        row = i * 8 + lane // 4
                        for j in range(8):
                            for kk in range(2):
                                index = j * 8 + (lane % 4) * 2 + kk
                                i1 = j // 2
                                i3 = (i * 8) % 64 // 16
                                i4 = i % 2
                                i5 = j % 2
                                fragment[i1, 0, i3, i4, i5, kk] = smem[row, index]
                    packed = _pack_fragment_literal(fragment.reshape(-1), 3)
                    for i in range(4):
                        row = by * 4 + e * (k // 16) + i
                        for kk in range(4):
                            col = bx * 128 + lane * 4 + kk
                            out[row, col] = packed[i * 4 + kk]
    return (out & 0xFFFFFFFF).astype(np.uint32).view(np.int32).reshape(e_count, k // 16, 2 * n)


def repack_closed_form(codes: np.ndarray) -> np.ndarray:
    """Vectorised packed-weight layout, equal to :func:`repack_literal`.

    Word ``c`` of packed row ``kb``: ``nb = c // 128``, ``t = (c % 128) // 4``,
    ``s = c % 4``; for ``rh, kh, kk`` in {0, 1} the code of weight
    ``(n, k) = (64 nb + 16 s + 8 rh + t // 4, 16 kb + 8 kh + 2 (t % 4) + kk)`` sits
    at bit ``4 (2 rh + kh) + 16 kk``.
    """
    codes = np.asarray(codes).astype(np.uint32)
    e_count, n, k = codes.shape
    assert n % 64 == 0 and k % 16 == 0
    # [E, nb, s, rh, r8, kb, kh, q, kk]
    v = codes.reshape(e_count, n // 64, 4, 2, 8, k // 16, 2, 4, 2)
    # -> [E, kb, nb, r8, q, s, rh, kh, kk]
    v = v.transpose(0, 5, 1, 4, 7, 2, 3, 6, 8)
    word = np.zeros(v.shape[:-3], dtype=np.uint32)
    for rh in range(2):
        for kh in range(2):
            for kk in range(2):
                word |= (v[..., rh, kh, kk] & 0xF) << np.uint32(4 * (2 * rh + kh) + 16 * kk)
    # column = 128 nb + 4 (4 r8 + q) + s
    return word.reshape(e_count, k // 16, 2 * n).view(np.int32)


def unpack_closed_form(packed: np.ndarray, n: int, k: int) -> np.ndarray:
    """Inverse of :func:`repack_closed_form`: int32 [E, K/16, 2N] -> codes [E, N, K]."""
    w = np.asarray(packed).view(np.uint32)
    e_count = w.shape[0]
    w = w.reshape(e_count, k // 16, n // 64, 8, 4, 4)  # [E, kb, nb, r8, q, s]
    out = np.zeros((e_count, n // 64, 4, 2, 8, k // 16, 2, 4, 2), dtype=np.int32)
    for rh in range(2):
        for kh in range(2):
            for kk in range(2):
                nib = (w >> np.uint32(4 * (2 * rh + kh) + 16 * kk)) & 0xF
                # nib [E, kb, nb, r8, q, s] -> out[E, nb, s, rh, r8, kb, kh, q, kk]
                out[:, :, :, rh, :, :, kh, :, kk] = nib.transpose(0, 2, 5, 3, 1, 4)
    return out.reshape(e_count, n, k)


def permute_scale(scale: torch.Tensor) -> torch.Tensor:
    """bf16 [E, N, K/32] -> [E, K/32, N] with the 64-column lane permutation:
    ``out[e, g, 64c + j] = scale[e, 64c + 8 (j % 8) + j // 8, g]``.

    Follows chord_kernels/operator/packing.py:45-52 (``_pack_weight_scale``).
    """
    e_count, n, groups = scale.shape
    j = torch.arange(64)
    src = 8 * (j % 8) + j // 8
    t = scale.transpose(1, 2).contiguous()  # [E, G, N]
    t = t.view(e_count, groups, n // 64, 64)[..., src]
    return t.reshape(e_count, groups, n).contiguous()


# --------------------------------------------------------------------- routing --

def topk_ids_random(num_tokens: int, top_k: int, num_experts: int,
                    generator: torch.Generator) -> torch.Tensor:
    """``top_k`` distinct experts per token: score every expert, keep the top.

    Follows tests/generators.py:174-189 (``generate_topk_ids``, "random").
    """
    scores = torch.randn((num_tokens, num_experts), dtype=torch.float32, generator=generator)
    return scores.topk(top_k, dim=1)[1].to(torch.int32)


def align_routing_blocks(topk_ids: torch.Tensor, block_m: int, num_experts: int,
                         expert_base: int = 0, allow_empty: bool = True):
    """CPU ``moe_align_block_size``: routes sorted by expert into ``block_m``
    blocks, each a valid prefix padded with the sentinel ``numel``; experts
    without routes emit no block.

    Follows tests/generators.py:192-230 (``align_routing_blocks``); adds the
    expert-parallel window ``[expert_base, expert_base + num_experts)`` that
    docs/getting_started.md:21 describes ("EP routing may carry only this rank's
    routes") and, unlike the reference generator, returns an empty routing
    instead of raising when nothing is routed here.
    """
    flat = topk_ids.reshape(-1).to(torch.int64)
    sentinel = flat.numel()
    parts, experts = [], []
    for local in range(num_experts):
        rows = torch.where(flat == local + expert_base)[0]
        if rows.numel() == 0:
            continue
        blocks = math.ceil(rows.numel() / block_m)
        rows = torch.nn.functional.pad(rows, (0, blocks * block_m - rows.numel()), value=sentinel)
        parts.append(rows)
        experts.extend([local] * blocks)
    if not parts:
        if not allow_empty:
            raise ValueError("routing produced no active expert blocks")
        return (torch.zeros(0, dtype=torch.int32), torch.zeros(0, dtype=torch.int32),
                torch.tensor(0, dtype=torch.int32))
    sorted_ids = torch.cat(parts).to(torch.int32).contiguous()
    expert_ids = torch.tensor(experts, dtype=torch.int32)
    return sorted_ids, expert_ids, torch.tensor(sorted_ids.numel(), dtype=torch.int32)


# ------------------------------------------------------------------------ GEMMs --

def dequantize_bf16(codes: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """``RN_bf16((code - 8) * scale)``: codes int [..., N, K], scale bf16
    [..., N, K/32] -> bf16 [..., N, K].

    Follows tests/generators.py:302-311 (the dequantisation inside
    ``reference_indexed``), which mirrors the kernels' ``lop3 -> sub -> mul``
    (include/humming/arith/mainloop_arith.cuh:85-100).
    """
    n, k = codes.shape[-2], codes.shape[-1]
    grouped = (codes - 8).to(torch.bfloat16).reshape(*codes.shape[:-1], k // GROUP, GROUP)
    return (grouped * scale.unsqueeze(-1)).reshape(*codes.shape[:-2], n, k)


def reference_indexed(activation: torch.Tensor, codes: torch.Tensor, scale: torch.Tensor,
                      topk_ids: torch.Tensor, top_k: int, projection: str = "gate_up",
                      expert_base: int = 0) -> torch.Tensor:
    """FP32 result of the routed GEMM, one row per route (row = route id).

    Follows tests/generators.py:259-319 (``reference_indexed``): BF16
    dequantisation, FP32 accumulation; gate_up reads token ``route // top_k``,
    down reads row ``route``.  Routes to experts outside
    ``[expert_base, expert_base + E)`` yield NaN rows (the kernel leaves them
    untouched).  Experts are processed one at a time so each is dequantised once.
    """
    route_experts = topk_ids.reshape(-1).to(torch.int64) - expert_base
    routes = route_experts.numel()
    inputs = activation if projection == "down" else activation.repeat_interleave(top_k, dim=0)
    out = torch.full((routes, codes.size(1)), float("nan"), dtype=torch.float32)
    for e in range(codes.size(0)):
        rows = torch.where(route_experts == e)[0]
        if rows.numel() == 0:
            continue
        w = dequantize_bf16(codes[e], scale[e]).float()
        out[rows] = inputs[rows].float() @ w.t()
    return out


def reference_indexed_rowwise(activation, codes, scale, topk_ids, top_k, projection="gate_up",
                              max_rows=None):
    """Literal restatement of ``reference_indexed`` (tests/generators.py:259-319):
    four routes at a time, einsum over re-dequantised experts.  Used to pin the
    per-expert form above and as the timed CPU baseline for small cases."""
    route_experts = topk_ids.reshape(-1).to(torch.int64)
    inputs = activation if projection == "down" else activation.repeat_interleave(top_k, dim=0)
    rows = route_experts.numel() if max_rows is None else min(max_rows, route_experts.numel())
    rows = max(rows, 1)
    route_experts = route_experts[:rows]
    inputs = inputs[:rows]
    out = torch.empty((rows, codes.size(1)), dtype=torch.float32)
    for start in range(0, rows, 4):
        end = min(start + 4, rows)
        expert = route_experts[start:end]
        deq = dequantize_bf16(codes[expert], scale[expert])
        out[start:end] = torch.einsum("rk,rnk->rn", inputs[start:end].float(), deq.float())
    return out


def _dequantize_f32(codes: torch.Tensor, scale: torch.Tensor, dequant: str) -> torch.Tensor:
    """FP32 weights of one expert: ``"bf16"`` rounds ``(code - 8) * scale`` to BF16 first
    (what the kernels compute), ``"fp32"`` does not (what the reference's grouped tests
    compare against, tests/test_w4a16_grouped.py:74-82)."""
    if dequant == "bf16":
        return dequantize_bf16(codes, scale).float()
    if dequant == "fp32":
        return dequant_reference_fp32(codes, scale)
    raise ValueError(f"dequant must be 'bf16' or 'fp32', got {dequant!r}")


def reference_contiguous(x2: torch.Tensor, codes: torch.Tensor, scale: torch.Tensor,
                         m_indices: torch.Tensor, block: int = 128, dequant: str = "bf16") -> torch.Tensor:
    """FP32 ``D[r] = x2[r] . deq(W[m_indices[tile first row]])^T`` per 128-row tile;
    tiles whose first row has index < 0 stay NaN (not written).  Padding rows inside a
    computed tile come out as the product of their (zeroed) activations, i.e. zeros.

    Follows the contiguous scheduler (include/deep_gemm/scheduler/gemm.cuh:273-274,
    include/deep_gemm/impls/sm90_w4a16_gemm.cuh:237-238) with the BF16
    dequantisation the kernels use (include/deep_gemm/ptx/ld_st.cuh:15-40), and the
    per-expert reference of tests/test_w4a16_grouped.py:225-241 (``dequant="fp32"``).
    """
    m = x2.size(0)
    out = torch.full((m, codes.size(1)), float("nan"), dtype=torch.float32)
    cache = {}
    for start in range(0, m, block):
        e = int(m_indices[start])
        if e < 0:
            continue
        if e not in cache:
            cache[e] = _dequantize_f32(codes[e], scale[e], dequant)
        out[start:start + block] = x2[start:start + block].float() @ cache[e].t()
    return out


def reference_masked(x3: torch.Tensor, codes: torch.Tensor, scale: torch.Tensor,
                     masked_m: torch.Tensor, dequant: str = "bf16") -> torch.Tensor:
    """FP32 ``D[g, :masked_m[g]] = x3[g, :masked_m[g]] . deq(W[g])^T``; other rows NaN.

    Follows chord_kernels/operator/grouped/api.py:116-133 (contract) and
    tests/test_w4a16_grouped.py:190-196 (per-group reference, ``dequant="fp32"``); the
    default is the BF16 dequantisation the kernels use.
    """
    g_count, max_m, _ = x3.shape
    out = torch.full((g_count, max_m, codes.size(1)), float("nan"), dtype=torch.float32)
    for g in range(g_count):
        mm = min(int(masked_m[g]), max_m)
        if mm <= 0:
            continue
        w = _dequantize_f32(codes[g], scale[g], dequant)
        out[g, :mm] = x3[g, :mm].float() @ w.t()
    return out


def dequant_reference_fp32(codes: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """FP32 dequantisation without the BF16 rounding of ``(code - 8) * scale``.

    Follows tests/test_w4a16_grouped.py:74-82 (``_dequant_reference``); the
    grouped tests compare against this looser form.
    """
    n, k = codes.shape
    signed = codes.float() - 8.0
    return (signed.reshape(n, k // GROUP, GROUP) * scale.float().reshape(n, k // GROUP, 1)).reshape(n, k)


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` in FP32, rounded once to BF16; gate is the first half
    of the columns (fused w13 convention, tests/generators.py:419-420)."""
    inter = gate_up.size(-1) // 2
    g = gate_up[..., :inter].float()
    u = gate_up[..., inter:].float()
    return (torch.nn.functional.silu(g) * u).to(torch.bfloat16)


# ---------------------------------------------------------------------- metrics --

def cosine_diff(actual: torch.Tensor, reference: torch.Tensor) -> float:
    """``1 - 2 sum(ab) / sum(a^2 + b^2)`` (tests/roofline.py:74-85)."""
    a, b = actual.double(), reference.double()
    den = (a.square() + b.square()).sum()
    if den.item() == 0:
        return 0.0
    return float(1 - (2 * (a * b).sum() / den).item())


def max_abs_rel(actual: torch.Tensor, reference: torch.Tensor) -> float:
    """``max|a - b| / max|b|``: the BF16-output tolerance metric (<= 1e-2)."""
    a, b = actual.double(), reference.double()
    den = b.abs().max().item()
    return float((a - b).abs().max().item() / den) if den else float((a - b).abs().max().item())


def traffic_bytes(active_experts: int, n: int, k: int, input_rows: int, output_rows: int) -> int:
    """Algorithmic DRAM bytes of one launch (tests/roofline.py:58-71)."""
    return (active_experts * n * (k // 2) + active_experts * n * (k // 32) * 2
            + input_rows * k * 2 + output_rows * n * 2)
