"""``indexed`` / ``indexed_block_m``: the routed (``moe_align_block_size``) W4A16
MoE GEMM, same interface as chord_kernels/ops.py:8-46 and
chord_kernels/operator/api.py:300-409, on the sm_100a tcgen05 kernel."""

from __future__ import annotations

import functools

import torch

from . import _checks, _lib
from .packing import PreparedWeight

MAX_BLOCK_M = 256

# Scratch the binder owns: per (device, stream) a zeroed lock buffer for calls that
# pass locks=None, and one status word per device.
_DEFAULT_LOCKS: dict[tuple[int, int], torch.Tensor] = {}
_STATUS: dict[int, torch.Tensor] = {}

_STATUS_BITS = {1: "producer wait", 2: "MMA-issuer wait", 4: "dequantisation wait",
                8: "epilogue wait", 16: "stream-K lock wait"}


def _device_index(device: torch.device) -> int:
    return device.index if device.index is not None else torch.cuda.current_device()


def _refuse_allocation_in_capture(device: torch.device, what: str) -> None:
    """A buffer created inside a stream capture would come from the graph's private
    pool and be handed out again after the graph is gone."""
    if torch.cuda.is_current_stream_capturing():
        raise RuntimeError(
            f"{what} would have to be allocated inside a CUDA-graph capture; "
            "pass your own zeroed locks tensor to captured calls and run one call on "
            f"{device} before capturing")


def status_word(device: torch.device) -> torch.Tensor:
    """Device word a kernel ORs an error code into when it gives up on a bounded
    wait (instead of hanging).  Zero in normal operation; :func:`check_status` reads it."""
    index = _device_index(device)
    word = _STATUS.get(index)
    if word is None:
        _refuse_allocation_in_capture(device, "the status word")
        word = torch.zeros(1, dtype=torch.int32, device=device)
        _STATUS[index] = word
    return word


def check_status(device=None) -> None:
    """Synchronise ``device`` and raise ``RuntimeError`` if any kernel since the last
    check gave up on a bounded wait (its output is then not to be trusted).  Clears the
    word.  After a stream-K lock timeout the caller's ``locks`` tensor must be zeroed
    again before it is reused."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    word = _STATUS.get(_device_index(device))
    if word is None:
        return
    torch.cuda.synchronize(device)
    bits = int(word.item())
    if bits:
        word.zero_()
        names = [name for bit, name in _STATUS_BITS.items() if bits & bit]
        raise RuntimeError(f"a chord_b200 kernel gave up on a bounded wait ({', '.join(names)}; "
                           f"status {bits})")


def default_locks(device: torch.device) -> torch.Tensor:
    key = (_device_index(device), torch.cuda.current_stream(device).cuda_stream)
    locks = _DEFAULT_LOCKS.get(key)
    if locks is None:
        _refuse_allocation_in_capture(device, "the default locks buffer (locks=None)")
        locks = torch.zeros(1024, dtype=torch.int32, device=device)
        _DEFAULT_LOCKS[key] = locks
    return locks


def gemm_scratch(device: torch.device, tile_tokens: int, locks: torch.Tensor | None,
                 sorted_len: int = 0, k: int = 0):
    """(locks, workspace) for one GEMM launch.  The workspace (FP32 stream-K partials
    and, for `indexed` with large routing blocks, the slot-ordered copy of the routed
    rows) comes from torch's caching allocator on every call, as in the reference's
    launcher (csrc/launcher/launcher.cpp:110-123): stream-ordered and graph-pool safe."""
    need_words, ws_bytes = _scratch_sizes(_device_index(device), tile_tokens, sorted_len, k,
                                          _lib.options_epoch())
    if locks is None:
        locks = default_locks(device)
    elif locks.numel() < need_words:
        raise RuntimeError(
            f"locks has {locks.numel()} lock words, this launch needs at least {need_words}"
        )
    workspace = torch.empty(ws_bytes // 4, dtype=torch.float32, device=device)
    return locks, workspace, ws_bytes


@functools.lru_cache(maxsize=256)
def _scratch_sizes(device_index: int, tile_tokens: int, sorted_len: int, k: int, options_epoch: int):
    """(lock words, workspace bytes) of a launch, asked of the library once per shape,
    device and option setting (the current device must be ``device_index``)."""
    del device_index, options_epoch  # cache keys only
    lib = _lib.load()
    need_words = lib.chord_b200_gemm_lock_words()
    if sorted_len > 0:
        ws_bytes = lib.chord_b200_indexed_workspace_bytes(tile_tokens, sorted_len, k)
    else:
        ws_bytes = lib.chord_b200_gemm_workspace_bytes(tile_tokens)
    if need_words < 0 or ws_bytes < 0:
        raise ValueError(_lib.last_error())
    return need_words, ws_bytes


def select_block_m(shape_n: int, shape_k: int, num_experts: int, routed_m: int) -> int:
    """Routing block size for a call; a multiple of 8 (here always a multiple of 16:
    the token dimension of a tile is the MMA's N, whose minimum is 16)."""
    _checks.integer("shape_n", shape_n, minimum=1)
    _checks.integer("shape_k", shape_k, minimum=1)
    _checks.integer("num_experts", num_experts, minimum=1)
    _checks.integer("routed_m", routed_m, minimum=0, type_error=True)
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
    _checks.tensor("inputs", inputs, nonempty=True)
    device = inputs.device
    _checks.supported_gpu(device)
    packed, scale, num_experts, shape_n, shape_k = _checks.prepared_weight(weight, device)
    if inputs.size(1) != shape_k:
        raise ValueError(f"inputs K={inputs.size(1)} does not match the weight's K={shape_k}")
    _checks.tensor("sorted_ids", sorted_ids, dtype=torch.int32, ndim=1, device=device)
    _checks.tensor("expert_ids", expert_ids, dtype=torch.int32, ndim=1, device=device)
    _checks.tensor("num_tokens_padded", num_tokens_padded, dtype=torch.int32, device=device)
    if num_tokens_padded.numel() != 1 or num_tokens_padded.ndim > 1:
        raise ValueError("num_tokens_padded must be a scalar or a one-element tensor")
    _checks.integer("top_k", top_k, minimum=1)
    routed_m = inputs.size(0) * top_k
    block_m = (select_block_m(shape_n, shape_k, num_experts, routed_m) if block_m is None
               else _checks.routing_block_m(block_m, MAX_BLOCK_M))
    if locks is not None:
        _checks.tensor("locks", locks, dtype=torch.int32, ndim=1, device=device)
    if outputs is None:
        outputs = torch.empty((routed_m, shape_n), dtype=torch.bfloat16, device=device)
    else:
        _checks.bf16_output(outputs, (routed_m, shape_n), device, exact_shape=True)
    if validate_routing:
        _checks.routing_contract(sorted_ids, expert_ids, num_tokens_padded, block_m, routed_m,
                                 num_experts)

    lib = _lib.load()
    with _lib.on_device(device):
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


def indexed_gate_up_silu(
    activation: torch.Tensor,
    weight: PreparedWeight,
    sorted_ids: torch.Tensor,
    expert_ids: torch.Tensor,
    num_tokens_padded: torch.Tensor,
    top_k: int,
    *,
    locks: torch.Tensor | None = None,
    outputs: torch.Tensor | None = None,
    block_m: int | None = None,
) -> torch.Tensor:
    """The gate_up projection with SiLU*mul applied in the GEMM's epilogue.

    ``weight`` is the fused w13 weight (``N`` rows: gate rows, then as many up rows).
    Returns BF16 ``[M * top_k, N / 2]`` with ``silu(gate) * up`` for every routed row,
    computed from the FP32 accumulators; rows no routed id names are left untouched.
    Arguments as for :func:`indexed`.  Where the fused kernel does not apply (routing
    blocks of 17 to 63 rows, or more than 128) the same result is produced by
    ``indexed`` followed by ``silu_mul`` (there rounded to BF16 in between).
    No counterpart in the reference, which leaves the activation to its caller.
    """
    from .fused_ops import silu_mul

    if not isinstance(activation, torch.Tensor) or activation.ndim != 2 or activation.dtype != torch.bfloat16:
        raise TypeError("inputs must be a 2D torch.bfloat16 tensor")
    _checks.tensor("inputs", activation, nonempty=True)
    device = activation.device
    _checks.supported_gpu(device)
    packed, scale, num_experts, shape_n, shape_k = _checks.prepared_weight(weight, device)
    if shape_n % 256:
        raise ValueError(f"a fused gate/up weight needs N divisible by 256, got {shape_n}")
    if activation.size(1) != shape_k:
        raise ValueError(f"inputs K={activation.size(1)} does not match the weight's K={shape_k}")
    _checks.integer("top_k", top_k, minimum=1)
    routed_m = activation.size(0) * top_k
    block_m = (select_block_m(shape_n, shape_k, num_experts, routed_m) if block_m is None
               else _checks.routing_block_m(block_m, MAX_BLOCK_M))
    inter = shape_n // 2
    if outputs is None:
        outputs = torch.empty((routed_m, inter), dtype=torch.bfloat16, device=device)
    else:
        _checks.bf16_output(outputs, (routed_m, inter), device, exact_shape=True)
    lib = _lib.load()
    if not lib.chord_b200_gate_up_silu_supported(shape_n, shape_k, block_m):
        gate_up = w4a16_indexed(activation, weight, sorted_ids, expert_ids, num_tokens_padded, top_k,
                                locks=locks, block_m=block_m)
        return silu_mul(gate_up, sorted_ids=sorted_ids, num_tokens_padded=num_tokens_padded,
                        outputs=outputs)
    _checks.tensor("sorted_ids", sorted_ids, dtype=torch.int32, ndim=1, device=device)
    _checks.tensor("expert_ids", expert_ids, dtype=torch.int32, ndim=1, device=device)
    _checks.tensor("num_tokens_padded", num_tokens_padded, dtype=torch.int32, device=device)
    if locks is not None:
        _checks.tensor("locks", locks, dtype=torch.int32, ndim=1, device=device)
    with _lib.on_device(device):
        need_words = lib.chord_b200_gemm_lock_words()
        if locks is None:
            locks = default_locks(device)
        elif locks.numel() < need_words:
            raise RuntimeError(
                f"locks has {locks.numel()} lock words, this launch needs at least {need_words}")
        ws_bytes = lib.chord_b200_gate_up_silu_workspace_bytes(block_m, sorted_ids.numel(), shape_k)
        if ws_bytes < 0:
            raise ValueError(_lib.last_error())
        workspace = torch.empty(ws_bytes // 4, dtype=torch.float32, device=device)
        _lib.check(lib.chord_b200_indexed_gate_up_silu(
            activation.data_ptr(), packed.data_ptr(), scale.data_ptr(),
            sorted_ids.data_ptr(), sorted_ids.numel(), expert_ids.data_ptr(), expert_ids.numel(),
            num_tokens_padded.data_ptr(), outputs.data_ptr(),
            locks.data_ptr(), locks.numel(), workspace.data_ptr(), ws_bytes,
            status_word(device).data_ptr(),
            activation.size(0), shape_n, shape_k, num_experts, top_k, block_m,
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


__all__ = ["check_status", "indexed", "indexed_gate_up_silu", "indexed_block_m", "w4a16_indexed", "select_block_m", "status_word"]
