"""Build libmegaup.so (sm_100a CUDA + C ABI) in-tree with nvcc.

Run as ``python -m megaup_b200.build``; ``ensure_built()`` rebuilds only when a
source is newer than the library. nvcc cross-compiles without a GPU.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
INCLUDE = PACKAGE_DIR.parent / "include"
LIB_DIR = PACKAGE_DIR / "_lib"
LIB_PATH = LIB_DIR / "libmegaup.so"

SOURCES = (CSRC / "mup_api.cu",)
HEADERS = (CSRC / "mup_ptx.cuh", CSRC / "mup_gemm.cuh", INCLUDE / "megaup.h")

NVCC_FLAGS = (
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-O3",
    "-std=c++17",
    "-lineinfo",
    "-shared",
    "-Xcompiler",
    "-fPIC",
    "-cudart",
    "static",
)


def find_nvcc() -> str:
    candidates = [
        os.environ.get("NVCC"),
        shutil.which("nvcc"),
        "/usr/local/cuda/bin/nvcc",
    ]
    for candidate in candidates:
        if candidate and Path(candidate).exists():
            return candidate
    raise RuntimeError("nvcc not found; set NVCC or add it to PATH")


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    return any(path.stat().st_mtime > built for path in (*SOURCES, *HEADERS))


def build(verbose: bool = False, ptxas_info: bool = False) -> Path:
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    command = [find_nvcc(), *NVCC_FLAGS]
    if ptxas_info:
        command += ["-Xptxas", "-v"]
    command += ["-I", str(INCLUDE), "-o", str(LIB_PATH), *map(str, SOURCES)]
    if verbose:
        print(" ".join(command), flush=True)
    result = subprocess.run(command, capture_output=True, text=True)
    if verbose or result.returncode != 0:
        sys.stdout.write(result.stdout)
        sys.stderr.write(result.stderr)
    if result.returncode != 0:
        raise RuntimeError(f"nvcc failed with exit code {result.returncode}")
    return LIB_PATH


def ensure_built() -> Path:
    if is_stale():
        build()
    return LIB_PATH


if __name__ == "__main__":
    build(verbose=True, ptxas_info="--ptxas-info" in sys.argv)
    print(f"built {LIB_PATH}")
