"""Builds the C-ABI shared library `libfastmoe_b200.so` in-tree with nvcc.

The library is plain CUDA C++ (no PyTorch headers), compiled for sm_100a only.
`python -m fastmoe_b200.build` rebuilds it; `ensure_built()` rebuilds only when a
source is newer than the library.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
LIB_PATH = PKG_DIR / "libfastmoe_b200.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-shared",
    "-Xcompiler",
    "-fPIC",
]


def _nvcc() -> str | None:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if cand and os.path.exists(cand) else None


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    return any(d.stat().st_mtime > built for d in deps)


def build(verbose: bool = False, force: bool = True) -> Path:
    """Compiles every .cu under csrc/ into one shared library. Raises on failure."""
    if not force and not _stale():
        return LIB_PATH
    nvcc = _nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build libfastmoe_b200.so")
    cmd = [nvcc, *NVCC_FLAGS, *os.environ.get("FASTMOE_B200_NVCC_FLAGS", "").split()]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    tmp = LIB_PATH.with_suffix(".so.tmp")
    cmd += ["-o", str(tmp), *map(str, sources())]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed ({proc.returncode}):\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


def ensure_built() -> Path:
    """Returns the library path, building it first if it is missing or stale and nvcc exists."""
    if _stale():
        if _nvcc() is None:
            if LIB_PATH.exists():
                return LIB_PATH  # no compiler on this machine: use the shipped binary
            raise RuntimeError(
                "libfastmoe_b200.so is missing and nvcc is not available to build it"
            )
        build(force=True)
    return LIB_PATH


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv)
    print(path)
