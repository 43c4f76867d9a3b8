"""In-tree build of the native libraries (no setuptools, no JIT cache).

Two shared objects are produced next to this file:

* ``libtilefusion_b200.so`` -- the CUDA kernels and the C-ABI declared in
  ``include/tilefusion_b200.h``; compiled by ``nvcc`` for sm_100a only.  It
  has no torch dependency and does not link ``libcuda``.
* ``libtilefusion_b200_torch.so`` -- the operator layer: ``TORCH_LIBRARY``
  registration of ``tilefusion::flash_attention`` (same schema as TileFusion's
  ``include/kernels/kernel_list.hpp:25-30``) and the added decode operators,
  each a thin call into the C-ABI.

Run ``python -m tilefusion_b200.build`` to (re)build both.
"""

from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
LIB_NAME = "libtilefusion_b200.so"
BIND_NAME = "libtilefusion_b200_torch.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--compiler-options", "-fPIC,-fvisibility=hidden",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found; the kernels cannot be built")
    return exe


def _source_hash(sources: list[Path], extra: str = "") -> str:
    h = hashlib.sha256(extra.encode())
    for s in sources:
        h.update(s.name.encode())
        h.update(s.read_bytes())
    return h.hexdigest()


def _up_to_date(target: Path, digest: str) -> bool:
    """True when `target` was built from sources with this digest (recorded in
    a side file, so the answer does not depend on file times, which a copy of
    the tree to another machine does not preserve)."""
    stamp = target.with_suffix(target.suffix + ".srchash")
    return target.exists() and stamp.exists() and stamp.read_text().strip() == digest


def _record(target: Path, digest: str) -> None:
    target.with_suffix(target.suffix + ".srchash").write_text(digest + "\n")


class _BuildLock:
    """Serialises builds between processes (ranks of one job import together)."""

    def __enter__(self):
        self._f = open(PKG_DIR / ".build.lock", "w")
        fcntl.flock(self._f, fcntl.LOCK_EX)
        return self

    def __exit__(self, *exc):
        fcntl.flock(self._f, fcntl.LOCK_UN)
        self._f.close()


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(
            "build step failed:\n  " + " ".join(cmd) + "\n" + proc.stdout + proc.stderr
        )


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile the kernels + C-ABI into ``libtilefusion_b200.so``."""
    out = PKG_DIR / LIB_NAME
    sources = [CSRC / "api.cu", CSRC / "registry.cc", CSRC / "shard.cc"]
    deps = sources + sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + [
        INCLUDE / "tilefusion_b200.h"
    ]
    digest = _source_hash(deps, " ".join(NVCC_FLAGS))
    if not force and _up_to_date(out, digest):
        return out
    with _BuildLock():
        if not force and _up_to_date(out, digest):
            return out
        tmp = out.with_suffix(".so.tmp")
        cmd = [_nvcc(), *NVCC_FLAGS, f"-I{INCLUDE}", f"-I{CSRC}", "-shared", "-o", str(tmp), "-ldl"]
        if verbose:
            cmd += ["-Xptxas", "-v"]
        cmd += [str(s) for s in sources]
        _run(cmd)
        os.replace(tmp, out)
        _record(out, digest)
    return out


def build_torch_binding(force: bool = False) -> Path:
    """Compile the TORCH_LIBRARY operator layer against the installed torch."""
    import torch
    from torch.utils import cpp_extension

    out = PKG_DIR / BIND_NAME
    src = CSRC / "torch_bind.cc"
    deps = [src, INCLUDE / "tilefusion_b200.h"]
    digest = _source_hash(deps, torch.__version__)
    if not force and _up_to_date(out, digest):
        return out
    torch_lib = Path(torch.__file__).resolve().parent / "lib"
    inc = []
    for p in cpp_extension.include_paths("cuda"):
        inc += ["-isystem", p]
    cxx = os.environ.get("CXX", "g++")
    cmd = [
        cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
        f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
        f"-I{INCLUDE}", *inc, str(src), "-o", str(out.with_suffix(".so.tmp")),
        f"-L{PKG_DIR}", "-ltilefusion_b200", f"-L{torch_lib}",
        "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda", "-lc10_cuda",
        "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}",
    ]
    with _BuildLock():
        if not force and _up_to_date(out, digest):
            return out
        _run(cmd)
        os.replace(out.with_suffix(".so.tmp"), out)
        _record(out, digest)
    return out


def build_all(force: bool = False) -> None:
    build_library(force=force)
    build_torch_binding(force=force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("built", PKG_DIR / LIB_NAME, "and", PKG_DIR / BIND_NAME)
