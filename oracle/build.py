"""TEST INFRASTRUCTURE - build the oracle's C kernel (oracle/ulysses_oracle.c) with gcc.

The target ISA is fixed (AVX2 + FMA) rather than -march=native, so a library
built on one machine runs on another.
"""

from __future__ import annotations

import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
SOURCE = HERE / "ulysses_oracle.c"
OUT_DIR = HERE / "_build"
LIB_PATH = OUT_DIR / "libulysses_oracle.so"


def build(verbose: bool = False) -> Path:
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    command = [
        "gcc", "-O3", "-mavx2", "-mfma", "-fopenmp", "-shared", "-fPIC",
        "-o", str(LIB_PATH), str(SOURCE),
    ]
    if verbose:
        print(" ".join(command), flush=True)
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        sys.stderr.write(result.stderr)
        raise RuntimeError(f"gcc failed with exit code {result.returncode}")
    return LIB_PATH


def ensure_built() -> Path:
    if not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < SOURCE.stat().st_mtime:
        build()
    return LIB_PATH


if __name__ == "__main__":
    print(build(verbose=True))
