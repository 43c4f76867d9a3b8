"""The C-ABI from a plain C program (no Python, no torch in the call path)."""

import shutil
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_c_caller(tmp_path, native_lib):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    exe = tmp_path / "cabi_smoke"
    libdir = ROOT / "tilefusion_b200"
    build = subprocess.run(
        [nvcc, "-x", "cu", str(ROOT / "tests" / "cabi_smoke.c"), f"-I{ROOT / 'include'}", f"-L{libdir}",
         "-ltilefusion_b200", "-Xlinker", f"-rpath={libdir}", "-o", str(exe)],
        capture_output=True, text=True)
    assert build.returncode == 0, build.stdout + build.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0 and run.stdout.strip().endswith("ok"), run.stdout + run.stderr
