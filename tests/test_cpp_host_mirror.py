"""The C++ host mirror (include/cogni_qmm.hpp) compiles as C++17 against the C ABI and behaves
like the reference's QuantMatmul module on the paths that need no GPU: block geometry, argument
checks and the error text for unsupported tensor types."""
import os
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.skipif(shutil.which("g++") is None, reason="g++ not found")
def test_host_mirror_compiles_and_checks(tmp_path):
    lib_dir = ROOT / "cogni_ml_b200"
    assert (lib_dir / "libcogni_qmm.so").exists(), "build the library first (python cogni_ml_b200/build.py)"
    exe = tmp_path / "host_mirror_check"
    env = {k: v for k, v in os.environ.items() if k not in ("CC", "CXX")}
    subprocess.run(["g++", "-std=c++17", "-Wall", "-Wextra", "-Werror", "-I", str(ROOT / "include"),
                    str(ROOT / "tests" / "cpp" / "host_mirror_check.cpp"), "-o", str(exe),
                    "-L", str(lib_dir), "-lcogni_qmm", f"-Wl,-rpath,{lib_dir}"],
                   check=True, env=env, capture_output=True, text=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True, env=env)
    assert out.returncode == 0 and out.stdout.strip().endswith("ok"), out.stdout + out.stderr
