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
# the same sources with -DMMF_EXPERIMENTS: configuration overrides (mmf_tuning) and the phase trace; loaded only by the
# configuration-sweep tests and by kernel experiments, never by the package itself
EXPERIMENTS_LIB_PATH = PKG_DIR / "libmmfree_b200_experiments.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC",
    "--threads", "0",
]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _digest(extra: str = "") -> str:
    h = hashlib.sha256()
    for p in sources() + sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h")):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(extra.encode())
    return h.hexdigest()


def _stamp(lib: Path) -> Path:
    return lib.with_suffix(".stamp")


def is_current(lib: Path = LIB_PATH, extra: str = "") -> bool:
    """True when the built library matches the sources it sits beside."""
    return lib.exists() and _stamp(lib).exists() and _stamp(lib).read_text().strip() == _digest(extra)


def _compile(lib: Path, defines: list[str], force: bool, verbose: bool) -> Path:
    extra = " ".join(defines)
    if not force and is_current(lib, extra):
        return lib
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError(f"nvcc not found: {lib.name} cannot be built on this machine")
    digest = _digest(extra)     # of the sources as they are NOW: an edit made while nvcc runs must trigger the next build
    tmp = lib.with_suffix(".so.tmp")
    cmd = [nvcc, *NVCC_FLAGS, *defines, "-I", str(INCLUDE), "-o", str(tmp), *map(str, sources())]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed ({proc.returncode}):\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        print(proc.stderr)
    os.replace(tmp, lib)
    _stamp(lib).write_text(digest + "\n")
    return lib


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile every .cu under csrc/ into the product shared library with nvcc. Idempotent."""
    return _compile(LIB_PATH, [], force, verbose)


def build_experiments_library(force: bool = False, verbose: bool = False) -> Path:
    """The experiments build (-DMMF_EXPERIMENTS) beside the product library. Idempotent."""
    return _compile(EXPERIMENTS_LIB_PATH, ["-DMMF_EXPERIMENTS"], force, verbose)


if __name__ == "__main__":
    import sys
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_experiments_library(force="--force" in sys.argv, verbose=False))
