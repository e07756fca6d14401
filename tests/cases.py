"""Seeded synthetic inputs shared by the tests, ``__graft_entry__.smoke()`` and
``bench.py``.  Distributions follow the benchmark definition: BF16 activations
N(0, 1), INT4 codes uniform in [0, 15] (value = code - 8), BF16 group-32 scales
uniform in [0.005, 0.02]; routing as tests/generators.py:140-230 of the reference
(top-k of N(0,1) scores, experts outside the local window dropped)."""

from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

from oracle import w4a16_oracle as O


def make_weights(num_experts, n, k, seed, lo=0.005, hi=0.02):
    g = torch.Generator().manual_seed(seed)
    codes = torch.randint(0, 16, (num_experts, n, k), dtype=torch.int32, generator=g)
    scale = (torch.rand((num_experts, n, k // 32), generator=g) * (hi - lo) + lo).to(torch.bfloat16)
    return codes, scale


def make_checkpoint_weights(num_experts, n, k, seed, lo=0.005, hi=0.02):
    """Random weights directly in checkpoint form (eight nibbles per int32 word)."""
    g = torch.Generator().manual_seed(seed)
    words = torch.randint(-2**31, 2**31 - 1, (num_experts, n, k // 8), dtype=torch.int64,
                          generator=g).to(torch.int32)
    scale = (torch.rand((num_experts, n, k // 32), generator=g) * (hi - lo) + lo).to(torch.bfloat16)
    return words, scale


def make_indexed_case(num_experts, n, k, m, top_k, block_m, seed, *, experts_total=None,
                      expert_base=0, projection="gate_up"):
    """Returns a dict with CPU tensors: codes, scale, x, topk_ids, routing."""
    codes, scale = make_weights(num_experts, n, k, seed)
    g = torch.Generator().manual_seed(seed + 100)
    rows = m * top_k if projection == "down" else m
    x = torch.randn((rows, k), generator=g).to(torch.bfloat16)
    topk = O.topk_ids_random(m, top_k, experts_total or num_experts, g)
    sorted_ids, expert_ids, padded = O.align_routing_blocks(topk, block_m, num_experts, expert_base)
    return dict(codes=codes, scale=scale, x=x, topk_ids=topk, sorted_ids=sorted_ids,
                expert_ids=expert_ids, num_tokens_padded=padded, top_k=top_k, block_m=block_m,
                expert_base=expert_base, projection=projection)


def make_masked_case(groups, max_m, n, k, expected_m, seed):
    codes, scale = make_weights(groups, n, k, seed)
    g = torch.Generator().manual_seed(seed + 7)
    x3 = torch.randn((groups, max_m, k), generator=g).to(torch.bfloat16)
    masked_m = torch.poisson(torch.full((groups,), float(expected_m)), generator=g)
    masked_m = masked_m.clamp(0, max_m).to(torch.int32)
    return dict(codes=codes, scale=scale, x3=x3, masked_m=masked_m, expected_m=expected_m)


def make_contiguous_case(counts, n, k, seed, extra_padding_tiles=0):
    """``counts[e]`` valid rows for expert e, each run padded to 128 (zeroed rows,
    index -1); optionally whole padding tiles at the end."""
    codes, scale = make_weights(len(counts), n, k, seed)
    g = torch.Generator().manual_seed(seed + 9)
    idx = []
    for e, c in enumerate(counts):
        pad = (c + 127) // 128 * 128
        idx += [e] * c + [-1] * (pad - c)
    idx += [-1] * (128 * extra_padding_tiles)
    m_indices = torch.tensor(idx, dtype=torch.int32)
    x2 = torch.randn((len(idx), k), generator=g).to(torch.bfloat16)
    x2[m_indices < 0] = 0
    return dict(codes=codes, scale=scale, x2=x2, m_indices=m_indices)


def load_grouped_golden(name):
    """One case of tests/golden/grouped.npz: inputs and expected BF16 outputs built by the
    reference's own ``make_masked_case`` / ``make_contiguous_case`` on the CPU."""
    z = np.load(Path(__file__).resolve().parent / "golden" / "grouped.npz")

    def bf16(key):
        return torch.from_numpy(z[f"{name}_{key}"].copy()).view(torch.bfloat16)

    shape = [int(v) for v in z[f"{name}_shape"]]
    n, k = shape[-2], shape[-1]
    groups = shape[0]
    codes = torch.from_numpy(O.unpack_checkpoint_uint4(z[f"{name}_checkpoint"])).reshape(groups, n, k)
    case = dict(codes=codes, scale=bf16("scale"), x=bf16("x"), ref=bf16("ref"), n=n, k=k, groups=groups,
                cosine_limit=float(z["cosine_limit"]))
    if name.startswith("masked"):
        case.update(max_m=shape[1], expected_m=shape[2],
                    masked_m=torch.from_numpy(z[f"{name}_masked_m"].copy()))
    else:
        case.update(m_indices=torch.from_numpy(z[f"{name}_m_indices"].copy()),
                    bounds=[tuple(int(v) for v in b) for b in z[f"{name}_bounds"]])
    return case
