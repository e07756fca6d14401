"""``indexed`` / ``indexed_block_m``: the routed (``moe_align_block_size``) W4A16
MoE GEMM, same interface as chord_kernels/ops.py:8-46 and
chord_kernels/operator/api.py:300-409, on the sm_100a tcgen05 kernel."""

from __future__ import annotations

import torch

from . import _lib
from .packing import PreparedWeight, _validate_supported_architecture

MAX_BLOCK_M = 256

# Scratch the binder owns, per (device, stream): a zeroed lock buffer for calls
# that pass locks=None, and one status word per device.
_DEFAULT_LOCKS: dict[tuple[int, int], torch.Tensor] = {}
_STATUS: dict[int, torch.Tensor] = {}


def _device_index(device: torch.device) -> int:
    return device.index if device.index is not None else torch.cuda.current_device()


def status_word(device: torch.device) -> torch.Tensor:
    """Device word a kernel ORs an error code into when it gives up on a bounded
    wait (instead of hanging).  Zero in normal operation; read it after a
    synchronize when debugging."""
    index = _device_index(device)
    word = _STATUS.get(index)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=device)
        _STATUS[index] = word
    return word


def default_locks(device: torch.device) -> torch.Tensor:
    key = (_device_index(device), torch.cuda.current_stream(device).cuda_stream)
    locks = _DEFAULT_LOCKS.get(key)
    if locks is None:
        locks = torch.zeros(1024, dtype=torch.int32, device=device)
        _DEFAULT_LOCKS[key] = locks
    return locks


def gemm_scratch(device: torch.device, tile_tokens: int, locks: torch.Tensor | None,
                 sorted_len: int = 0, k: int = 0):
    """(locks, workspace) for one GEMM launch.  The workspace (FP32 stream-K partials
    and, for `indexed` with large routing blocks, the slot-ordered copy of the routed
    rows) comes from torch's caching allocator on every call, as in the reference's
    launcher (csrc/launcher/launcher.cpp:110-123): stream-ordered and graph-pool safe."""
    lib = _lib.load()
    need_words = lib.chord_b200_gemm_lock_words()
    if locks is None:
        locks = default_locks(device)
    elif locks.numel() < need_words:
        raise RuntimeError(
            f"locks has {locks.numel()} lock words, this launch needs at least {need_words}"
        )
    if sorted_len > 0:
        ws_bytes = lib.chord_b200_indexed_workspace_bytes(tile_tokens, sorted_len, k)
    else:
        ws_bytes = lib.chord_b200_gemm_workspace_bytes(tile_tokens)
    if ws_bytes < 0:
        raise ValueError(_lib.last_error())
    workspace = torch.empty(ws_bytes // 4, dtype=torch.float32, device=device)
    return locks, workspace, ws_bytes


def _check_cuda_int32(name: str, tensor: torch.Tensor, device: torch.device) -> None:
    if not isinstance(tensor, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor, got {type(tensor).__name__}")
    if tensor.dtype != torch.int32:
        raise TypeError(f"{name} must be torch.int32, got {tensor.dtype}")
    if tensor.device != device or not tensor.is_contiguous():
        raise ValueError(f"{name} must be contiguous and on {device}")


def _validate_prepared_weight(weight: PreparedWeight, device: torch.device):
    """Same checks as chord_kernels/operator/api.py:233-248."""
    if not isinstance(weight, PreparedWeight):
        raise TypeError("weight must be a PreparedWeight from pack_w4a16()")
    n, k, e = weight.n, weight.k, weight.num_experts
    packed, scale = weight.packed, weight.scale
    if packed.dtype != torch.int32 or tuple(packed.shape) != (e, k // 16, n * 2):
        raise ValueError(f"packed weight must be int32 {(e, k // 16, n * 2)}, got {tuple(packed.shape)}")
    if scale.dtype != torch.bfloat16 or tuple(scale.shape) != (e, k // 32, n):
        raise ValueError(f"packed scale must be BF16 {(e, k // 32, n)}, got {tuple(scale.shape)}")
    if packed.device != device or scale.device != device:
        raise ValueError(f"weight must be on {device}, got {packed.device}")
    if not packed.is_contiguous() or not scale.is_contiguous():
        raise ValueError("packed weight and scale must be contiguous")
    return packed, scale, e, n, k


def _validate_routing(sorted_ids, expert_ids, num_tokens_padded, block_m, routed_limit, num_experts):
    """Synchronizing check of the routing contract (``validate_routing=True``);
    same rules and messages as chord_kernels/operator/api.py:251-297."""
    padded_count = int(num_tokens_padded.reshape(-1)[0].item())
    if padded_count < 0 or padded_count > sorted_ids.numel():
        raise ValueError(
            f"num_tokens_padded must be in [0, {sorted_ids.numel()}], got {padded_count}"
        )
    if padded_count % block_m:
        raise ValueError(
            f"num_tokens_padded must be a multiple of block_m={block_m}, got {padded_count}"
        )
    active_blocks = padded_count // block_m
    if expert_ids.numel() < active_blocks:
        raise ValueError(
            f"expert_ids must cover {active_blocks} active blocks, got {expert_ids.numel()}"
        )
    if not padded_count:
        return
    ids = sorted_ids[:padded_count]
    experts = expert_ids[:active_blocks]
    valid = ids.view(-1, block_m) < routed_limit
    route_ids = torch.sort(ids[(ids >= 0) & (ids < routed_limit)]).values
    if route_ids.numel() > 1:
        unique = bool((route_ids[1:] != route_ids[:-1]).all().item())
    else:
        unique = True
    if not bool((ids >= 0).all().item()):
        raise ValueError("sorted_ids values must be non-negative")
    if bool((valid & ((~valid).cumsum(dim=1) > 0)).any().item()):
        raise ValueError(
            "each active sorted_ids block must hold its routed ids as a prefix "
            "followed only by sentinels"
        )
    if not bool(((experts >= 0) & (experts < num_experts)).all().item()):
        raise ValueError(f"expert_ids values must be in [0, {num_experts - 1}]")
    if not unique:
        raise ValueError("active sorted_ids contains duplicate routed ids")


def select_block_m(shape_n: int, shape_k: int, num_experts: int, routed_m: int) -> int:
    """Routing block size for a call; a multiple of 8 (here always a multiple of 16:
    the token dimension of a tile is the MMA's N, whose minimum is 16)."""
    for name, value in (("shape_n", shape_n), ("shape_k", shape_k), ("num_experts", num_experts)):
        if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
            raise ValueError(f"{name} must be a positive int, got {value!r}")
    if isinstance(routed_m, bool) or not isinstance(routed_m, int):
        raise TypeError(f"routed_m must be an int, got {type(routed_m).__name__}")
    if routed_m < 0:
        raise ValueError(f"routed_m must be non-negative, got {routed_m}")
    return int(_lib.load().chord_b200_indexed_block_m(shape_n, shape_k, num_experts, routed_m))


def indexed_block_m(weight: PreparedWeight, num_tokens: int, top_k: int, *, device=None,
                    total_experts: int | None = None) -> int:
    """Routing block size ``indexed`` uses; align ``moe_align_block_size`` to it.

    For down pass gate/up's ``top_k`` here (the kernel call takes ``top_k=1``).
    Same signature as chord_kernels/operator/api.py:300-315, plus one optional
    keyword: under expert parallelism ``weight`` holds only this rank's experts while
    the router spreads ``num_tokens * top_k`` routes over ``total_experts``; naming the
    total lets the block size follow the rows this rank will really see (the
    reference folds that knowledge into per-deployment tuning tables,
    chord_kernels/operator/tuning.py:496-504).
    """
    if not isinstance(weight, PreparedWeight):
        raise TypeError("weight must be a PreparedWeight from pack_w4a16()")
    del device  # one schedule family: the block size does not depend on the GPU
    routed = num_tokens * top_k
    if total_experts is not None:
        if isinstance(total_experts, bool) or not isinstance(total_experts, int) or total_experts < weight.num_experts:
            raise ValueError(
                f"total_experts must be an int >= the weight's {weight.num_experts} experts, got {total_experts!r}"
            )
        routed = -(-routed * weight.num_experts // total_experts)
    return select_block_m(weight.n, weight.k, weight.num_experts, routed)


def w4a16_indexed(
    inputs: torch.Tensor,
    weight: PreparedWeight,
    sorted_ids: torch.Tensor,
    expert_ids: torch.Tensor,
    num_tokens_padded: torch.Tensor,
    top_k: int,
    *,
    locks: torch.Tensor | None = None,
    outputs: torch.Tensor | None = None,
    block_m: int | None = None,
    validate_routing: bool = False,
) -> torch.Tensor:
    """BF16 x INT4 group-32 indexed MoE GEMM; see :func:`indexed`.

    Checks and exception classes follow chord_kernels/operator/api.py:336-384.
    """
    if not isinstance(inputs, torch.Tensor) or inputs.ndim != 2 or inputs.dtype != torch.bfloat16:
        raise TypeError("inputs must be a 2D torch.bfloat16 tensor")
    if not inputs.is_cuda or not inputs.is_contiguous() or 0 in inputs.shape:
        raise ValueError("inputs must be a non-empty contiguous CUDA tensor")
    device = inputs.device
    _validate_supported_architecture(device)
    packed, scale, num_experts, shape_n, shape_k = _validate_prepared_weight(weight, device)
    if inputs.size(1) != shape_k:
        raise ValueError(f"inputs K={inputs.size(1)} does not match the weight's K={shape_k}")
    for name, tensor in (("sorted_ids", sorted_ids), ("expert_ids", expert_ids),
                         ("num_tokens_padded", num_tokens_padded)):
        _check_cuda_int32(name, tensor, device)
    if sorted_ids.ndim != 1 or expert_ids.ndim != 1:
        raise ValueError("sorted_ids and expert_ids must be 1D")
    if num_tokens_padded.numel() != 1 or num_tokens_padded.ndim > 1:
        raise ValueError("num_tokens_padded must be a scalar or a one-element tensor")
    if isinstance(top_k, bool) or not isinstance(top_k, int) or top_k <= 0:
        raise ValueError(f"top_k must be a positive int, got {top_k!r}")

    routed_m = inputs.size(0) * top_k
    if block_m is None:
        block_m = select_block_m(shape_n, shape_k, num_experts, routed_m)
    elif isinstance(block_m, bool) or not isinstance(block_m, int) or block_m <= 0 or block_m % 8:
        raise ValueError(f"routing block_m must be a positive multiple of 8, got {block_m!r}")
    elif block_m > MAX_BLOCK_M:
        raise ValueError(f"routing block_m must be at most {MAX_BLOCK_M}, got {block_m}")

    if locks is not None:
        _check_cuda_int32("locks", locks, device)
        if locks.ndim != 1:
            raise ValueError("locks must be 1D")
    if outputs is None:
        outputs = torch.empty((routed_m, shape_n), dtype=torch.bfloat16, device=device)
    else:
        if not isinstance(outputs, torch.Tensor) or outputs.dtype != torch.bfloat16:
            raise TypeError("outputs must be a torch.bfloat16 tensor")
        if (tuple(outputs.shape) != (routed_m, shape_n) or outputs.device != device
                or not outputs.is_contiguous()):
            raise ValueError(
                f"outputs must be contiguous BF16 {(routed_m, shape_n)} on {device}, "
                f"got {tuple(outputs.shape)}"
            )
    if validate_routing:
        _validate_routing(sorted_ids, expert_ids, num_tokens_padded, block_m, routed_m, num_experts)

    lib = _lib.load()
    with torch.cuda.device(device):
        locks, workspace, ws_bytes = gemm_scratch(device, block_m, locks, sorted_ids.numel(), shape_k)
        _lib.check(lib.chord_b200_indexed(
            inputs.data_ptr(), packed.data_ptr(), scale.data_ptr(),
            sorted_ids.data_ptr(), sorted_ids.numel(), expert_ids.data_ptr(), expert_ids.numel(),
            num_tokens_padded.data_ptr(), outputs.data_ptr(),
            locks.data_ptr(), locks.numel(), workspace.data_ptr(), ws_bytes,
            status_word(device).data_ptr(),
            inputs.size(0), shape_n, shape_k, num_experts, top_k, block_m,
            _lib.stream_handle(device),
        ))
    return outputs


def indexed(
    activation,
    weight,
    sorted_ids,
    expert_ids,
    num_tokens_padded,
    top_k: int,
    *,
    locks=None,
    outputs=None,
    block_m: int | None = None,
    validate_routing: bool = False,
):
    """Indexed (``moe_align_block_size``-routed) BF16 x INT4 MoE GEMM.

    ``activation`` is BF16 ``[M, K]`` and ``weight`` comes from ``pack_w4a16``.
    The routing must be aligned to ``indexed_block_m(weight, num_tokens, top_k)``;
    a host that aligns one routing for both projections passes that block size as
    ``block_m``.  ``locks`` is a zeroed int32 tensor of 1024 words: every launch
    indexes it from word 0 and leaves it zeroed, so launches that are ordered (one
    stream, one graph) share it, while launches that may run concurrently each
    need their own; with ``locks=None`` a per-stream buffer owned by the library is
    used.  Returns BF16 ``[M * top_k, N]``; rows no routed id names are left
    untouched.  For the down projection pass the routed activations and
    ``top_k=1``.  Same signature as chord_kernels/ops.py:8-46.
    """
    return w4a16_indexed(
        activation, weight, sorted_ids, expert_ids, num_tokens_padded, top_k,
        locks=locks, outputs=outputs, block_m=block_m, validate_routing=validate_routing,
    )


__all__ = ["indexed", "indexed_block_m", "w4a16_indexed", "select_block_m", "status_word"]
