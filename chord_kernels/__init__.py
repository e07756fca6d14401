"""``chord_kernels`` import name for code written against the reference library
(chord_kernels/__init__.py:6-21): the same five callables, served by chord_b200."""

from typing import Any

__all__ = [
    "contiguous",
    "indexed",
    "indexed_block_m",
    "masked",
    "pack_w4a16",
]


def __getattr__(name: str) -> Any:
    if name in __all__:
        import chord_b200

        value = getattr(chord_b200, name)
        globals()[name] = value
        return value
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__() -> list[str]:
    return sorted(set(globals()) | set(__all__))
