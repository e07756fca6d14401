"""Generates tests/golden/*.npz by running the reference's own CPU-runnable code.

Run once in a container that has a read-only checkout of the reference:

    CHORD_REFERENCE=<path to the checkout> python tests/golden/make_golden.py

What it runs, unmodified, from the reference:
  * tests/generators.py: ``generate_topk_ids``, ``align_routing_blocks``,
    ``reference_indexed``, ``pack_checkpoint_uint4``
  * chord_kernels/operator/packing.py: ``_pack_weight_scale``
  * tests/test_w4a16_grouped.py: ``_dequant_reference``, and for ``grouped.npz``
    ``make_masked_case`` / ``make_contiguous_case`` on ``device="cpu"``: the inputs
    and the expected outputs of the reference's own masked and contiguous tests
  * tests/roofline.py: ``traffic_bytes``, ``error_metrics``
The reference's packer itself (``repack_w4a16``) is a CUDA kernel and cannot run
without a GPU, so the packed-weight layout has no golden vector here.

Inputs are seeded and small (E=4, N=256, K=512, 32 tokens, top_k=2, and the
reference's tiny 8x128x128 E=4 case); the codes are stored only in checkpoint form
(eight nibbles per word) and outputs as raw integer views, so the fixtures are exact
and stay a few hundred KB.
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch

OUT = Path(__file__).resolve().parent


def reference_root() -> Path:
    root = os.environ.get("CHORD_REFERENCE") or (sys.argv[1] if len(sys.argv) > 1 else None)
    if not root or not (Path(root) / "chord_kernels").is_dir():
        raise SystemExit("set CHORD_REFERENCE (or pass the path) to a checkout of the reference")
    return Path(root)


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().copy()


def grouped_cases(gen) -> None:
    """Inputs and expected outputs of the reference's masked / contiguous tests
    (tests/test_w4a16_grouped.py:168-242), small shapes, CPU.  Masked: groups whose
    valid-row count reaches max_m next to partial ones, and a second case with a few
    rows per group.  Contiguous: experts shorter than their 128-row run (trailing -1
    rows, zeroed activations) and a case with two full blocks per expert."""
    import test_w4a16_grouped as grouped  # reference tests/test_w4a16_grouped.py

    cpu = torch.device("cpu")
    arrays = {}
    masked = {"masked_a": grouped.MaskedCase(4, 32, 30, 128, 256),
              "masked_b": grouped.MaskedCase(3, 64, 8, 256, 128)}
    for name, case in masked.items():
        a3, codes, scale, masked_m, ref = grouped.make_masked_case(case, cpu)
        arrays[f"{name}_shape"] = np.array([case.num_groups, case.max_m, case.expected_m_per_group,
                                            case.n, case.k], dtype=np.int64)
        arrays[f"{name}_x"] = bf16_bits(a3)
        arrays[f"{name}_checkpoint"] = gen.pack_checkpoint_uint4(codes).numpy()
        arrays[f"{name}_scale"] = bf16_bits(scale)
        arrays[f"{name}_masked_m"] = masked_m.numpy()
        arrays[f"{name}_ref"] = bf16_bits(ref)
    contiguous = {"contiguous_a": grouped.ContiguousCase(3, 100, 128, 256),
                  "contiguous_b": grouped.ContiguousCase(2, 256, 256, 128)}
    for name, case in contiguous.items():
        a2, codes, scale, m_indices, ref, bounds = grouped.make_contiguous_case(case, cpu)
        arrays[f"{name}_shape"] = np.array([case.num_groups, case.expected_m_per_group, case.n,
                                            case.k], dtype=np.int64)
        arrays[f"{name}_x"] = bf16_bits(a2)
        arrays[f"{name}_checkpoint"] = gen.pack_checkpoint_uint4(codes).numpy()
        arrays[f"{name}_scale"] = bf16_bits(scale)
        arrays[f"{name}_m_indices"] = m_indices.numpy()
        arrays[f"{name}_ref"] = bf16_bits(ref)
        arrays[f"{name}_bounds"] = np.array(bounds, dtype=np.int64)
    arrays["cosine_limit"] = np.array(grouped._COSINE_LIMIT)
    np.savez_compressed(OUT / "grouped.npz", **arrays)
    print("grouped written", (OUT / "grouped.npz").stat().st_size, "bytes")


def main() -> None:
    reference = reference_root()
    sys.path.insert(0, str(reference / "tests"))
    sys.path.insert(0, str(reference))
    os.environ.setdefault("CHORD_CACHE_DIR", "/tmp/chord_cache")
    os.environ.setdefault("CHORD_TMP_DIR", "/tmp/chord_tmp")
    import generators as gen  # reference tests/generators.py
    import roofline  # reference tests/roofline.py
    from chord_kernels.operator.packing import _pack_weight_scale

    cpu = torch.device("cpu")
    for name, (e, n, k, m, top_k, block_m, seed) in {
        "mid": (4, 256, 512, 32, 2, 16, 20260901),
        "tiny": (4, 128, 128, 8, 1, 8, 7),
    }.items():
        g = torch.Generator(device=cpu).manual_seed(seed)
        x = torch.randn((m, k), dtype=torch.bfloat16, generator=g)
        codes = torch.randint(0, 16, (e, n, k), dtype=torch.int32, generator=g)
        scale = (torch.rand((e, n, k // 32), dtype=torch.float32, generator=g) * 0.015 + 0.005
                 ).to(torch.bfloat16)
        rg = torch.Generator(device=cpu).manual_seed(m)
        topk = gen.generate_topk_ids(num_tokens=m, top_k=top_k, num_experts=e, device=cpu,
                                     generator=rg, distribution="random")
        sorted_ids, expert_ids, padded = gen.align_routing_blocks(
            topk, block_m=block_m, num_experts=e)
        ref_gate_up, _ = gen.reference_indexed(x, codes, scale, topk, top_k, projection="gate_up")
        x_routed = torch.randn((m * top_k, k), dtype=torch.bfloat16, generator=g)
        ref_down, _ = gen.reference_indexed(x_routed, codes, scale, topk, top_k, projection="down")
        packed_scale = _pack_weight_scale(scale)
        checkpoint = gen.pack_checkpoint_uint4(codes)
        # _dequant_reference of the grouped tests (FP32, no BF16 rounding), expert 0 only
        signed = codes[0].float() - 8.0
        deq0 = (signed.reshape(n, k // 32, 32) * scale[0].float().reshape(n, k // 32, 1)).reshape(n, k)
        np.savez_compressed(
            OUT / f"{name}.npz",
            shape=np.array([e, n, k, m, top_k, block_m], dtype=np.int64),
            x=bf16_bits(x), x_routed=bf16_bits(x_routed),
            scale=bf16_bits(scale), topk_ids=topk.numpy(), sorted_ids=sorted_ids.numpy(),
            expert_ids=expert_ids.numpy(), num_tokens_padded=np.array(int(padded)),
            ref_gate_up=ref_gate_up.numpy().view(np.int32), ref_down=ref_down.numpy().view(np.int32),
            packed_scale=bf16_bits(packed_scale), checkpoint=checkpoint.numpy(),
            dequant_fp32_e0=deq0.numpy().view(np.int32),
            traffic=np.array(roofline.traffic_bytes(e, n, k, m, m * top_k), dtype=np.int64),
            cos_self=np.array(roofline.error_metrics(ref_gate_up, ref_gate_up)[0]),
        )
        print(name, "written", (OUT / f"{name}.npz").stat().st_size, "bytes")
    grouped_cases(gen)


if __name__ == "__main__":
    main()
