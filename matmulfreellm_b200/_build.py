"""In-tree build of libmmfree_b200.so (hand-written CUDA, sm_100a only).

The shared library is compiled next to this file so that it travels with the source tree;
nothing is installed into site-packages and no JIT cache is used.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
LIB_PATH = PKG_DIR / "libmmfree_b200.so"
STAMP_PATH = PKG_DIR / "libmmfree_b200.stamp"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC",
    "--threads", "0",
]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _digest() -> str:
    h = hashlib.sha256()
    for p in sources() + sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h")):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    """True when the built library matches the sources it sits beside."""
    return LIB_PATH.exists() and STAMP_PATH.exists() and STAMP_PATH.read_text().strip() == _digest()


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile every .cu under csrc/ into one shared library with nvcc. Idempotent."""
    if not force and is_current():
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: libmmfree_b200.so cannot be built on this machine")
    tmp = LIB_PATH.with_suffix(".so.tmp")
    cmd = [nvcc, *NVCC_FLAGS, "-I", str(INCLUDE), "-o", str(tmp), *map(str, sources())]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed ({proc.returncode}):\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        print(proc.stderr)
    os.replace(tmp, LIB_PATH)
    STAMP_PATH.write_text(_digest() + "\n")
    return LIB_PATH


if __name__ == "__main__":
    import sys
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
