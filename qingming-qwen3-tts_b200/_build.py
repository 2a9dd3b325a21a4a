"""Compiles the CUDA sources under csrc/ into lib/libqm_attention_b200.so (sm_100a only).

nvcc cross-compiles without a GPU, so this also serves as the "does it build"
check on a CPU-only machine.  The library is built in-tree so that it travels
with the source tree to the machine that runs it.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
LIB_DIR = PACKAGE_DIR / "lib"
LIB_PATH = LIB_DIR / "libqm_attention_b200.so"
HEADER = PACKAGE_DIR.parent / "include" / "qm_attention.h"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-shared",
]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    deps = sources() + sorted(CSRC.glob("*.cuh")) + [HEADER]
    return any(p.stat().st_mtime > built for p in deps)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Builds the shared library if it is missing or older than its sources."""
    if not force and not is_stale():
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; cannot build libqm_attention_b200.so")
    LIB_DIR.mkdir(exist_ok=True)
    cmd = [nvcc, *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", str(LIB_PATH), *map(str, sources()), "-ldl"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    if verbose:
        print(proc.stdout + proc.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force=True, verbose=True))
