"""chord_b200: W4A16 MoE expert GEMMs for NVIDIA B200 (sm_100a).

Drop-in for the public surface of the reference's ``chord_kernels`` package
(chord_kernels/__init__.py:6-21): ``pack_w4a16``, ``indexed``,
``indexed_block_m``, ``contiguous``, ``masked``.  Names resolve on first access,
so importing the package does not import torch.
"""

from importlib import import_module
from typing import Any

__all__ = [
    "contiguous",
    "indexed",
    "indexed_block_m",
    "masked",
    "pack_w4a16",
]

_EXPORTS = {
    "indexed": "chord_b200.indexed_gemm",
    "indexed_block_m": "chord_b200.indexed_gemm",
    "masked": "chord_b200.grouped_gemm",
    "contiguous": "chord_b200.grouped_gemm",
    "pack_w4a16": "chord_b200.packing",
    "PreparedWeight": "chord_b200.packing",
    "silu_mul": "chord_b200.fused_ops",
    "moe_align_block_size": "chord_b200.fused_ops",
    "check_status": "chord_b200.indexed_gemm",
    "indexed_gate_up_silu": "chord_b200.indexed_gemm",
    "set_option": "chord_b200._lib",
}


def __getattr__(name: str) -> Any:
    if name in _EXPORTS:
        value = getattr(import_module(_EXPORTS[name]), name)
        globals()[name] = value
        return value
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__() -> list[str]:
    return sorted(set(globals()) | set(__all__))
