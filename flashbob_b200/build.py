"""Build libbob_sm100.so in-tree with nvcc for sm_100a.

    python -m flashbob_b200.build

nvcc cross-compiles without a GPU.  The library lands next to this file so that it is found by
`flashbob_b200._lib` without any install step.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libbob_sm100.so"
SOURCES = ("api.cu", "selftest.cu", "noalloc.cu")
HEADERS = ("ptx.cuh", "sweep.cuh", "tmap.h", "internal.h")


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")
    return cand


def _stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = [CSRC / s for s in SOURCES + HEADERS if (CSRC / s).exists()]
    deps.append(PKG.parent / "include" / "bob_sm100.h")
    return any(d.stat().st_mtime > t for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile the CUDA sources into libbob_sm100.so (skipped when up to date)."""
    if not force and not _stale():
        return LIB
    srcs = [str(CSRC / s) for s in SOURCES if (CSRC / s).exists()]
    cmd = [
        _nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        "-shared", "-Xcompiler", "-fPIC", "-o", str(LIB), *srcs,
    ]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{res.stdout}\n{res.stderr}")
    if verbose:
        print(res.stderr)
    return LIB


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
