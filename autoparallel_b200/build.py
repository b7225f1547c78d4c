"""Builds libapk.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m autoparallel_b200.build [--force]
"""
from __future__ import annotations

import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent / "csrc"
SOURCES = [CSRC / "apk.cu"]
HEADERS = [
    CSRC / "gemm_kernel.cuh",
    CSRC / "collectives_kernel.cuh",
    CSRC / "ptx.cuh",
    CSRC.parent.parent / "include" / "apk.h",
]
OUT = CSRC / "libapk.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
    "-cudart", "static",
]


def _stale() -> bool:
    if not OUT.exists():
        return True
    t = OUT.stat().st_mtime
    return any(p.stat().st_mtime > t for p in SOURCES + HEADERS)


def build_native(force: bool = False, verbose: bool = False) -> Path:
    """Compile the CUDA library if it is missing or older than its sources."""
    if not force and not _stale():
        return OUT
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", str(OUT), *map(str, SOURCES)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
    if verbose:
        print(res.stderr)
    return OUT


if __name__ == "__main__":
    print(build_native(force="--force" in sys.argv, verbose="-v" in sys.argv))
