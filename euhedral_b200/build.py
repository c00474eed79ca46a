"""Builds libeuhedral_cuda.so (the sm_100a kernels and their C ABI) in-tree with nvcc.

    python -m euhedral_b200.build [--force]

nvcc cross-compiles without a GPU; the built library sits next to the sources so that it travels with the tree.
"""

from __future__ import annotations

import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
CSRC = PACKAGE / "csrc"
LIB_DIR = PACKAGE / "lib"
LIBRARY = LIB_DIR / "libeuhedral_cuda.so"
HEADER = PACKAGE.parent / "include" / "euhedral_cuda.h"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC,-fvisibility=hidden", "-cudart", "static",
]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + [HEADER]


def stale() -> bool:
    if not LIBRARY.exists():
        return True
    built = LIBRARY.stat().st_mtime
    return any(path.stat().st_mtime > built for path in sources())


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not stale():
        return LIBRARY
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    LIB_DIR.mkdir(exist_ok=True)
    command = [nvcc, *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", str(LIBRARY), str(CSRC / "abi.cu")]
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{result.stdout}\n{result.stderr}")
    if verbose:
        print(result.stderr)
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
