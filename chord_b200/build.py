"""Ahead-of-time build of ``libchord_b200.so`` (sm_100a only) with nvcc.

The reference compiles its kernels at run time through NVRTC
(chord_kernels/operator/jit/compiler.py:51-105); here every kernel is compiled
once, in-tree, and linked into one C-ABI shared library.  Run as
``python -m chord_b200.build``.
"""

from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
LIB_PATH = PACKAGE_DIR / "libchord_b200.so"
SOURCES = ("core.cu", "gemm.cu", "pack.cu", "fused.cu", "ep.cu")
ARCH_FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a")


def _nvcc() -> str:
    nvcc = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        raise RuntimeError("nvcc not found; set NVCC or put the CUDA toolkit on PATH")
    return nvcc


def _newest_source_mtime() -> float:
    files = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    files.append(PACKAGE_DIR.parent / "include" / "chord_b200.h")
    return max(f.stat().st_mtime for f in files if f.exists())


def is_fresh() -> bool:
    return LIB_PATH.exists() and LIB_PATH.stat().st_mtime >= _newest_source_mtime()


def _compile(nvcc: str, src: str, obj_dir: Path, verbose: bool) -> Path:
    obj = obj_dir / (src + ".o")
    cmd = [
        nvcc, *ARCH_FLAGS, "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
        "-Xptxas", "-v" if verbose else "-warn-spills",
        "-c", str(CSRC / src), "-o", str(obj),
    ]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        sys.stderr.write(proc.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the CUDA sources for sm_100a and link ``libchord_b200.so`` in-tree."""
    if not force and is_fresh():
        return LIB_PATH
    nvcc = _nvcc()
    obj_dir = PACKAGE_DIR / "build"
    obj_dir.mkdir(exist_ok=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        objs = list(pool.map(lambda s: _compile(nvcc, s, obj_dir, verbose), SOURCES))
    tmp = LIB_PATH.with_suffix(".so.tmp")
    cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp), *map(str, objs)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
