"""Builds libcogni_qmm.so (CUDA kernels + C ABI) in-tree with nvcc for sm_100a.

    python cogni_ml_b200/build.py          # build if sources are newer than the library
    python cogni_ml_b200/build.py --force

nvcc cross-compiles without a GPU, so this runs on a CPU-only build machine; the resulting
shared library sits beside this file and is what `cogni_ml_b200._lib` loads.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libcogni_qmm.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: cannot build libcogni_qmm.so")
    return exe


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def needs_build() -> bool:
    if not LIB_PATH.exists():
        return True
    newest = max(p.stat().st_mtime for p in list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh"))
                 + [PKG_DIR.parent / "include" / "cogni_qmm.h", PKG_DIR.parent / "include" / "cogni_qmm_diag.h"])
    return newest > LIB_PATH.stat().st_mtime


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return LIB_PATH
    cmd = [_nvcc(), *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", str(LIB_PATH), *map(str, sources()), "-ldl"]
    env = dict(os.environ)
    # the image exports CC/CXX pointing at a compiler wrapper nvcc cannot drive; use PATH's g++
    env.pop("CC", None)
    env.pop("CXX", None)
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
