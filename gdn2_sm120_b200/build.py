"""Compile the CUDA sources in ``csrc/`` into ``libgdn2_b200.so`` next to this file.

``nvcc`` cross-compiles for sm_100a without a GPU, so this runs anywhere the CUDA
toolkit is installed.  The shared object is built in-tree (it is git-ignored) and is
rebuilt only when a source or header is newer than it.

    python -m gdn2_sm120_b200.build [--force] [--verbose]
"""

from __future__ import annotations

import os
import pathlib
import shutil
import subprocess
import sys

PACKAGE_DIR = pathlib.Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
INCLUDE = PACKAGE_DIR.parent / "include"
LIB_NAME = "libgdn2_b200.so"
LIB_PATH = PACKAGE_DIR / LIB_NAME

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-shared", "-Xcompiler", "-fPIC",
    "-Xcompiler", "-Wall",
]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found; the gdn2_b200 kernels cannot be built")
    return found


def sources() -> list[pathlib.Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    return any(dep.stat().st_mtime > built for dep in deps)


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    if not force and not _stale():
        return LIB_PATH
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(INCLUDE)]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [str(src) for src in sources()]
    tmp = LIB_PATH.with_suffix(".so.tmp")
    cmd += ["-o", str(tmp), "-lcudart", "-lcuda"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed with exit code {proc.returncode}")
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
