"""Argument checks shared by ``pack_w4a16``, ``indexed``, ``masked`` and ``contiguous``.

The error contract is the reference's (chord_kernels/operator/packing.py:68-117,
operator/api.py:222-297 and 336-384, operator/grouped/api.py:24-73 and 134-245): a
wrong Python type or tensor dtype raises ``TypeError``, a wrong shape, device, layout
or value raises ``ValueError``, an unsupported GPU raises ``RuntimeError``, and every
message names the offending parameter.  The substrings the reference's own tests
match (``"routing block_m"``, ``"routed_m"``, ``"shape_n"``, ``"locks"``,
``"lock words"``; tests/test_w4a16_indexed.py:1033-1039, 1409-1411) are kept.
"""

from __future__ import annotations

import torch

SUPPORTED_COMPUTE_CAPABILITY_MAJOR = 10


_CHECKED_DEVICES: set = set()


def supported_gpu(device: torch.device) -> None:
    """This build runs on compute capability 10.x only (the reference gates on
    9.0 / 10.0 / 10.3, packing.py:16-23).  The verdict is remembered per device: the
    query costs microseconds on a path that is called once per GEMM."""
    if device in _CHECKED_DEVICES:
        return
    major, minor = torch.cuda.get_device_capability(device)
    if major == SUPPORTED_COMPUTE_CAPABILITY_MAJOR:
        _CHECKED_DEVICES.add(device)
    if major != SUPPORTED_COMPUTE_CAPABILITY_MAJOR:
        raise RuntimeError(
            "chord_b200 W4A16 kernels require an SM100/SM103 Blackwell GPU, got compute "
            f"capability {major}.{minor} on {device}"
        )


def tensor(name: str, value, *, dtype: torch.dtype | None = None, ndim: int | None = None,
           device: torch.device | None = None, cuda: bool = True, contiguous: bool = True,
           nonempty: bool = False) -> torch.Tensor:
    """One tensor argument: type and dtype first (``TypeError``), then placement,
    layout and extent (``ValueError``)."""
    if not isinstance(value, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor, got {type(value).__name__}")
    if dtype is not None and value.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {value.dtype}")
    if ndim is not None and value.ndim != ndim:
        raise ValueError(f"{name} must be {ndim}D, got shape {tuple(value.shape)}")
    if cuda and not value.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor, got device {value.device}")
    if device is not None and value.device != device:
        raise ValueError(f"{name} must be on {device}, got {value.device}")
    if contiguous and not value.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if nonempty and value.numel() == 0:
        raise ValueError(f"{name} must be non-empty, got shape {tuple(value.shape)}")
    return value


def integer(name: str, value, *, minimum: int | None = None, type_error: bool = False) -> int:
    """A Python int (``bool`` is refused) of at least ``minimum``.  ``type_error``
    selects the class raised for a non-int, as the reference differs per parameter."""
    if isinstance(value, bool) or not isinstance(value, int):
        message = f"{name} must be an int, got {value!r}"
        raise TypeError(message) if type_error else ValueError(message)
    if minimum is not None and value < minimum:
        bound = "positive" if minimum == 1 else ("non-negative" if minimum == 0 else f">= {minimum}")
        raise ValueError(f"{name} must be {bound}, got {value}")
    return value


def flag(name: str, value) -> bool:
    if not isinstance(value, bool):
        raise TypeError(f"{name} must be a bool, got {type(value).__name__}")
    return value


def routing_block_m(block_m, limit: int) -> int:
    if isinstance(block_m, bool) or not isinstance(block_m, int) or block_m <= 0 or block_m % 8:
        raise ValueError(f"routing block_m must be a positive multiple of 8, got {block_m!r}")
    if block_m > limit:
        raise ValueError(f"routing block_m must be at most {limit}, got {block_m}")
    return block_m


def prepared_weight(weight, device: torch.device, *, dtype_error=ValueError):
    """A :class:`PreparedWeight` whose tensors agree with its recorded ``n, k, E`` and
    live, contiguous, on ``device``.  Returns ``(packed, scale, E, n, k)``."""
    from .packing import PreparedWeight

    if not isinstance(weight, PreparedWeight):
        raise TypeError("weight must be a PreparedWeight from pack_w4a16()")
    n, k, e = weight.n, weight.k, weight.num_experts
    packed, scale = weight.packed, weight.scale
    if packed.dtype != torch.int32 or scale.dtype != torch.bfloat16:
        raise dtype_error(
            f"packed weight must be int32 and its scale bfloat16, got {packed.dtype} / {scale.dtype}")
    want_packed, want_scale = (e, k // 16, n * 2), (e, k // 32, n)
    if tuple(packed.shape) != want_packed or tuple(scale.shape) != want_scale:
        raise ValueError(
            f"packed weight {tuple(packed.shape)} / scale {tuple(scale.shape)} disagree with the "
            f"recorded n={n}, k={k}, num_experts={e}: expected {want_packed} / {want_scale}")
    for name, t in (("packed weight", packed), ("packed scale", scale)):
        if t.device != device:
            raise ValueError(f"{name} must be on {device}, got {t.device}")
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
    return packed, scale, e, n, k


def bf16_output(outputs, shape: tuple[int, int], device: torch.device, *, exact_shape: bool) -> torch.Tensor:
    """A caller-provided output buffer: BF16, contiguous, on ``device``, of ``shape``
    (or, for the grouped operators, of that many elements)."""
    if not isinstance(outputs, torch.Tensor) or outputs.dtype != torch.bfloat16:
        raise TypeError("outputs must be a torch.bfloat16 tensor")
    fits = tuple(outputs.shape) == shape if exact_shape else outputs.numel() == shape[0] * shape[1]
    if not fits or outputs.device != device or not outputs.is_contiguous():
        raise ValueError(
            f"outputs must be contiguous BF16 {shape} on {device}, got {tuple(outputs.shape)} "
            f"on {outputs.device}")
    return outputs


def routing_contract(sorted_ids, expert_ids, num_tokens_padded, block_m: int, routed_limit: int,
                     num_experts: int) -> None:
    """The indexed routing contract, checked on the device with one read-back
    (``validate_routing=True``; rules of operator/api.py:251-297): the padded count is
    a multiple of ``block_m`` within the buffers, ids are non-negative, every block is
    its routed ids followed only by sentinels, expert ids are in range and no routed
    id appears twice."""
    padded = int(num_tokens_padded.reshape(-1)[0].item())
    if padded < 0 or padded > sorted_ids.numel():
        raise ValueError(f"num_tokens_padded must be in [0, {sorted_ids.numel()}], got {padded}")
    if padded % block_m:
        raise ValueError(f"num_tokens_padded must be a multiple of block_m={block_m}, got {padded}")
    blocks = padded // block_m
    if expert_ids.numel() < blocks:
        raise ValueError(f"expert_ids must cover {blocks} active blocks, got {expert_ids.numel()}")
    if padded == 0:
        return
    ids = sorted_ids[:padded].view(blocks, block_m)
    routed = ids < routed_limit
    # A routed id after a sentinel inside a block: the running count of sentinels is
    # already positive where `routed` is still true.
    broken_prefix = (routed & ((~routed).cumsum(dim=1) > 0)).any()
    experts = expert_ids[:blocks]
    bad_expert = ((experts < 0) | (experts >= num_experts)).any()
    negative = (ids < 0).any()
    kept = torch.sort(ids[routed & (ids >= 0)]).values
    duplicate = (kept[1:] == kept[:-1]).any() if kept.numel() > 1 else negative.new_zeros(())
    verdict = torch.stack([negative, broken_prefix, bad_expert, duplicate]).cpu().tolist()
    if verdict[0]:
        raise ValueError("sorted_ids values must be non-negative")
    if verdict[1]:
        raise ValueError("each active sorted_ids block must hold its routed ids as a prefix "
                         "followed only by sentinels")
    if verdict[2]:
        raise ValueError(f"expert_ids values must be in [0, {num_experts - 1}]")
    if verdict[3]:
        raise ValueError("active sorted_ids contains duplicate routed ids")
