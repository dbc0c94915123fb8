"""Ahead-of-time build of the CUDA library (``python -m nvfp4_gemm_b200.build``).

Compiles ``csrc/nvfp4_api.cu`` for sm_100a into ``libnvfp4_b200.so`` next to this file.
nvcc cross-compiles without a GPU.  Nothing is JIT-compiled at call time (the reference
builds at import with ``load_inline``, s_128t.py:587-602).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
SRC = PKG_DIR / "csrc" / "nvfp4_api.cu"
LIB = PKG_DIR / "libnvfp4_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC",
    "-cudart", "static",
]


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found (looked on PATH and in $CUDA_HOME/bin)")
    return nvcc


def sources() -> list[Path]:
    return [SRC, *sorted((PKG_DIR / "csrc").glob("*.cuh")), PKG_DIR.parent / "include" / "nvfp4_b200.h"]


def needs_build() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    return any(s.stat().st_mtime > t for s in sources())


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return LIB
    tmp = LIB.with_suffix(".so.building")
    cmd = [find_nvcc(), *NVCC_FLAGS, "-o", str(tmp), str(SRC)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
        print(" ".join(cmd), file=sys.stderr)
    subprocess.check_call(cmd)
    os.replace(tmp, LIB)       # a reader never sees a half-written library
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
