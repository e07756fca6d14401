"""Golden vectors from the reference's own GPU kernels (needs a GPU and a checkout of
novitalabs/chord; not needed to run the tests, which read the committed .npz).

    python tests/golden/make_reference_gpu_golden.py --reference /path/to/chord \
        [--out tests/golden/reference_gpu.npz]

What it records, for seeded inputs generated here:
  * `pack_w4a16` of the reference (its repack kernel, NVRTC-compiled from
    chord_kernels/operator/include/humming/kernel/repack.cuh) for both input forms:
    the packed words and the permuted scales.  This pins the packed-weight layout to
    the reference's own output.
  * `indexed` of the reference (its Blackwell `mma.sync` schedule) on a small routed
    case: the BF16 output, with the routing it was given.
Nothing of the reference is copied: the script imports it from the path given.
"""

from __future__ import annotations

import argparse
import os
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def checkpoint_words(codes: torch.Tensor) -> torch.Tensor:
    """int32 [E, N, K] codes -> [E, N, K/8] words, eight little-endian nibbles per word."""
    e, n, k = codes.shape
    c = codes.to(torch.int64).reshape(e, n, k // 8, 8)
    words = torch.zeros((e, n, k // 8), dtype=torch.int64)
    for j in range(8):
        words |= c[..., j] << (4 * j)
    words = torch.where(words >= 2**31, words - 2**32, words)
    return words.to(torch.int32)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path to a checkout of the reference")
    ap.add_argument("--out", default=str(Path(__file__).resolve().parent / "reference_gpu.npz"))
    args = ap.parse_args()

    scratch = tempfile.mkdtemp(prefix="chord_ref_")
    os.environ.setdefault("CHORD_TMP_DIR", os.path.join(scratch, "tmp"))
    os.environ.setdefault("CHORD_CACHE_DIR", os.path.join(scratch, "cache"))
    os.makedirs(os.environ["CHORD_TMP_DIR"], exist_ok=True)
    os.makedirs(os.environ["CHORD_CACHE_DIR"], exist_ok=True)
    sys.path.insert(0, args.reference)
    import chord_kernels as ref  # the reference package

    from oracle import w4a16_oracle as O

    dev = torch.device("cuda:0")
    bits = lambda t: t.contiguous().view(torch.int16).cpu().numpy()  # noqa: E731
    out: dict[str, np.ndarray] = {}

    # ---- packing: E=3, N=256, K=320 (K an odd multiple of 64)
    g = torch.Generator().manual_seed(101)
    codes = torch.randint(0, 16, (3, 256, 320), generator=g, dtype=torch.int32)
    scale = (torch.rand((3, 256, 10), generator=g) * 0.015 + 0.005).to(torch.bfloat16)
    words = checkpoint_words(codes)
    from_codes = ref.pack_w4a16(codes.to(dev), scale.to(dev))
    from_words = ref.pack_w4a16(words.to(dev), scale.to(dev), packed=True)
    torch.cuda.synchronize()
    assert torch.equal(from_codes.packed, from_words.packed), "reference: the two input forms disagree"
    out["pack_words"] = words.numpy()
    out["pack_scale_in"] = bits(scale)
    out["pack_packed"] = from_words.packed.cpu().numpy()
    out["pack_scale_out"] = bits(from_words.scale)

    # ---- indexed: E=4, N=256, K=256, 32 tokens, top_k 2
    e, n, k, m, top_k = 4, 256, 256, 32, 2
    g = torch.Generator().manual_seed(202)
    icodes = torch.randint(0, 16, (e, n, k), generator=g, dtype=torch.int32)
    iscale = (torch.rand((e, n, k // 32), generator=g) * 0.015 + 0.005).to(torch.bfloat16)
    x = torch.randn((m, k), generator=g).to(torch.bfloat16)
    topk = O.topk_ids_random(m, top_k, e, g)
    weight = ref.pack_w4a16(icodes.to(dev), iscale.to(dev))
    block_m = int(ref.indexed_block_m(weight, m, top_k))
    sorted_ids, expert_ids, padded = O.align_routing_blocks(topk, block_m, e, 0)
    locks = torch.zeros(1024, dtype=torch.int32, device=dev)
    result = ref.indexed(x.to(dev), weight, sorted_ids.to(dev), expert_ids.to(dev),
                         padded.to(dev).reshape(1), top_k, locks=locks)
    torch.cuda.synchronize()
    assert bool((locks == 0).all())
    out["idx_shape"] = np.array([e, n, k, m, top_k, block_m], dtype=np.int32)
    out["idx_words"] = checkpoint_words(icodes).numpy()
    out["idx_scale"] = bits(iscale)
    out["idx_x"] = bits(x)
    out["idx_topk"] = topk.numpy().astype(np.int32)
    out["idx_sorted_ids"] = sorted_ids.numpy()
    out["idx_expert_ids"] = expert_ids.numpy()
    out["idx_num_tokens_padded"] = np.array([int(padded)], dtype=np.int32)
    out["idx_out"] = bits(result)
    np.savez_compressed(args.out, **out)
    print(f"wrote {args.out}: block_m {block_m}, packed {tuple(from_words.packed.shape)}, "
          f"indexed out {tuple(result.shape)}")



if __name__ == "__main__":
    main()
