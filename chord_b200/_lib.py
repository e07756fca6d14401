"""ctypes binding of ``libchord_b200.so`` (the C ABI declared in include/chord_b200.h).

Takes the place of the reference's torch-extension binder
(chord_kernels/operator/ops.py:46-147): there the native side is a torch C++
extension built on first use; here it is a prebuilt C-ABI library that sees raw
device pointers and a stream handle.  There is no fallback: if the library is
missing or a call fails, an exception is raised.
"""

from __future__ import annotations

import ctypes
import os
from pathlib import Path

_LIB = None
_LIB_PATH = Path(__file__).resolve().parent / "libchord_b200.so"

_i64 = ctypes.c_int64
_ptr = ctypes.c_void_p
_int = ctypes.c_int

# name -> (restype, argtypes); mirrors include/chord_b200.h one to one.
SIGNATURES = {
    "chord_b200_last_error": (ctypes.c_char_p, []),
    "chord_b200_version": (ctypes.c_char_p, []),
    "chord_b200_set_option": (_int, [ctypes.c_char_p, _i64]),
    "chord_b200_repack_w4a16": (_int, [_ptr, _ptr, _i64, _i64, _i64, _int, _ptr, _ptr]),
    "chord_b200_permute_scale": (_int, [_ptr, _ptr, _i64, _i64, _i64, _ptr]),
    "chord_b200_indexed_block_m": (_int, [_i64, _i64, _i64, _i64]),
    "chord_b200_masked_tile_m": (_int, [_i64]),
    "chord_b200_gemm_workspace_bytes": (_i64, [_i64]),
    "chord_b200_indexed_workspace_bytes": (_i64, [_i64, _i64, _i64]),
    "chord_b200_gemm_lock_words": (_int, []),
    "chord_b200_schedule_segments": (_i64, [_i64, _i64, _i64, _i64, _ptr, _i64]),
    "chord_b200_indexed": (_int, [_ptr, _ptr, _ptr, _ptr, _i64, _ptr, _i64, _ptr, _ptr, _ptr, _i64,
                                  _ptr, _i64, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _ptr]),
    "chord_b200_indexed_rows": (_int, [_ptr, _ptr, _ptr, _ptr, _i64, _ptr, _i64, _ptr, _ptr, _ptr, _i64,
                                       _ptr, _i64, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _ptr]),
    "chord_b200_indexed_slots": (_int, [_ptr, _ptr, _ptr, _ptr, _i64, _ptr, _i64, _ptr, _ptr, _ptr, _ptr, _i64,
                                        _ptr, _i64, _ptr, _i64, _i64, _i64, _i64, _i64, _int, _ptr]),
    "chord_b200_indexed_gate_up_silu": (_int, [_ptr, _ptr, _ptr, _ptr, _i64, _ptr, _i64, _ptr, _ptr, _ptr,
                                               _i64, _ptr, _i64, _ptr, _i64, _i64, _i64, _i64, _i64, _i64,
                                               _ptr]),
    "chord_b200_gate_up_silu_supported": (_int, [_i64, _i64, _i64]),
    "chord_b200_gate_up_silu_workspace_bytes": (_i64, [_i64, _i64, _i64]),
    "chord_b200_indexed_static_scratch": (_int, [_ptr, _ptr, _ptr, _ptr, _i64, _ptr, _i64, _ptr, _ptr,
                                                 _ptr, _i64, _ptr, _i64, _i64, _i64, _i64, _i64, _i64,
                                                 _ptr]),
    "chord_b200_contiguous": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _ptr, _i64, _ptr,
                                     _i64, _i64, _i64, _i64, _int, _ptr]),
    "chord_b200_masked": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _ptr, _i64, _ptr,
                                 _i64, _i64, _i64, _i64, _i64, _int, _ptr]),
    "chord_b200_silu_mul": (_int, [_ptr, _ptr, _i64, _i64, _ptr]),
    "chord_b200_silu_mul_routed": (_int, [_ptr, _ptr, _ptr, _i64, _ptr, _i64, _i64, _ptr]),
    "chord_b200_moe_align_block_size": (_int, [_ptr, _i64, _i64, _i64, _i64, _ptr, _i64, _ptr,
                                               _i64, _ptr, _ptr]),
    "chord_b200_ep_state_bytes": (_i64, []),
    "chord_b200_ep_plan": (_int, [_ptr, _i64, _i64, _i64, _i64, _ptr, _ptr, _i64, _ptr]),
    "chord_b200_ep_dispatch": (_int, [_ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _ptr, _ptr,
                                      _ptr, _ptr, _i64, _i64, _i64, _ptr]),
    "chord_b200_ep_align": (_int, [_ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _ptr, _i64, _ptr, _i64, _ptr,
                                   _ptr, _ptr, _i64, _i64, _ptr, _i64, _ptr]),
    "chord_b200_ep_combine_signal": (_int, [_ptr, _i64, _i64, _i64, _ptr]),
    "chord_b200_ep_combine_wait": (_int, [_ptr, _i64, _i64, _ptr]),
}


def library_path() -> Path:
    override = os.environ.get("CHORD_B200_LIB")
    return Path(override) if override else _LIB_PATH


def load() -> ctypes.CDLL:
    """Load the native library once; raise if it has not been built."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = library_path()
    if not path.exists():
        raise RuntimeError(
            f"{path} is missing: build it with `python -m chord_b200.build` "
            "(chord_b200 has no fallback path without its CUDA library)"
        )
    lib = ctypes.CDLL(str(path))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _LIB = lib
    _apply_env_options(lib)
    return lib


def _apply_env_options(lib: ctypes.CDLL) -> None:
    """Tuning overrides, the counterpart of the reference's ``CHORD_W4A16_*``
    variables (chord_kernels/operator/grouped/heuristics.py:32-39)."""
    for env, option in (
        ("CHORD_B200_XLOAD", "x_load"),
        ("CHORD_B200_DEQUANT_GROUPS", "dequant_groups"),
        ("CHORD_B200_MAX_STAGES", "max_stages"),
        ("CHORD_B200_GRID", "grid_limit"),
        ("CHORD_B200_KSPLIT", "ksplit"),
        ("CHORD_B200_PREGATHER", "pregather"),
        ("CHORD_B200_DECODE_KERNEL", "decode_kernel"),
        ("CHORD_B200_PDL", "pdl"),
        ("CHORD_B200_NPAIR", "npair"),
        ("CHORD_B200_PAIR", "pair"),
    ):
        value = os.environ.get(env)
        if value is None:
            continue
        if option == "x_load" and not value.isdigit():
            value = {"cpasync": "0", "gather4": "1"}[value]
        check(lib.chord_b200_set_option(option.encode(), int(value)))


def last_error() -> str:
    return load().chord_b200_last_error().decode(errors="replace")


def check(code: int) -> None:
    """Map a C-ABI return code to the exception class the reference raises."""
    if code == 0:
        return
    message = last_error()
    if code == 1:
        raise ValueError(message)
    raise RuntimeError(message)


_OPTIONS_EPOCH = 0


def options_epoch() -> int:
    """Changes whenever an option is set through this module (scratch sizes depend on
    some options, so caches of them are keyed by it)."""
    return _OPTIONS_EPOCH


def set_option(name: str, value: int) -> None:
    global _OPTIONS_EPOCH
    check(load().chord_b200_set_option(name.encode(), int(value)))
    _OPTIONS_EPOCH += 1


def stream_handle(device) -> int:
    import torch

    return torch.cuda.current_stream(device).cuda_stream


class on_device:
    """``with on_device(device):`` makes ``device`` current for the C-ABI calls inside;
    when it already is (the common case) nothing is switched, which saves the several
    microseconds a ``torch.cuda.device`` round trip costs per GEMM call."""

    __slots__ = ("guard",)

    def __init__(self, device):
        import torch

        index = device.index
        self.guard = None if index is None or index == torch.cuda.current_device() else torch.cuda.device(device)

    def __enter__(self):
        if self.guard is not None:
            self.guard.__enter__()

    def __exit__(self, *exc):
        if self.guard is not None:
            self.guard.__exit__(*exc)
