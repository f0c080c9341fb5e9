"""Builds oracle/_ref/: the reference's OWN CUDA GEMV kernels as loadable cubins.  TEST
INFRASTRUCTURE ONLY -- nothing under cogni_ml_b200/ may load what this makes.

The reference ships its CUDA path as PTX text (`.target sm_80`): three files under
src/ml/cuda/kernels/ and two heredocs inside Crystal sources.  `ptxas` assembles that text,
unmodified and read from where it lies in the reference checkout, into sm_100a cubins.  Only the
cubins (binaries) are written, and only into oracle/_ref/ (git-ignored); no reference source is
copied into this repository.  The cubins are what pins the CPU oracle: tests run the reference's
kernels and the oracle on the same seeded tensors and require agreement inside the reference's own
probe thresholds (bin/cuda_q4k_gemv_probe.cr:269-289, bin/cuda_q8_gemv_probe.cr:390).

    python oracle/make_ref.py [reference_root]

Without a reference checkout (e.g. on a GPU box that only received the built files) this does
nothing and the already-built cubins are used.
"""
from __future__ import annotations

import os
import re
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"

# cubin name -> (source file inside the reference, heredoc constant or None for a plain .ptx file)
SOURCES = {
    "q4k_gemv": ("src/ml/cuda/kernels/q4k_gemv_probe.ptx", None),
    "q5k_gemv": ("src/ml/cuda/kernels/q5k_gemv_probe.ptx", None),
    "q6k_gemv": ("src/ml/cuda/kernels/q6k_gemv_probe.ptx", None),
    "q4k_dual_gemv": ("src/ml/cuda/kernels/q4k_dual_gemv_probe.ptx", None),
    "q8_0_gemv": ("bin/cuda_q8_gemv_probe.cr", "PTX"),
    "output_top": ("src/ml/cuda/qwen_output_head_runner.cr", "TOP1_PTX"),
}


def reference_root(arg: str | None = None) -> Path | None:
    root = Path(arg or os.environ.get("COGNI_ML_REFERENCE", "/root/reference"))
    return root if (root / "src/ml/cuda/driver.cr").exists() else None


def _heredoc(text: str, const: str) -> str:
    """The body of `CONST = <<-PTX ... PTX` (Crystal strips the closing line's indentation)."""
    m = re.search(r"^\s*" + re.escape(const) + r"\s*=\s*<<-PTX\n(.*?)^\s*PTX\s*$", text, re.S | re.M)
    if not m:
        raise RuntimeError(f"heredoc {const} not found")
    return m.group(1)


def _ptxas() -> str:
    exe = shutil.which("ptxas") or "/usr/local/cuda/bin/ptxas"
    if not os.path.exists(exe):
        raise RuntimeError("ptxas not found")
    return exe


def build(root_arg: str | None = None, force: bool = False) -> list[Path]:
    root = reference_root(root_arg)
    if root is None:
        return sorted(OUT.glob("*.cubin"))
    OUT.mkdir(exist_ok=True)
    made = []
    with tempfile.TemporaryDirectory() as tmp:
        for name, (rel, const) in SOURCES.items():
            src = root / rel
            dst = OUT / f"{name}.cubin"
            made.append(dst)
            if not force and dst.exists() and dst.stat().st_mtime >= src.stat().st_mtime:
                continue
            ptx = src
            if const is not None:  # the PTX text sits inside a Crystal source: extract to scratch
                ptx = Path(tmp) / f"{name}.ptx"
                ptx.write_text(_heredoc(src.read_text(), const))
            subprocess.run([_ptxas(), "-arch=sm_100a", str(ptx), "-o", str(dst)], check=True,
                           capture_output=True)
    return made


if __name__ == "__main__":
    for p in build(sys.argv[1] if len(sys.argv) > 1 else None, force=True):
        print(p)
