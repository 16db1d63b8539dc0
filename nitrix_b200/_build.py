"""Builds the CUDA library in-tree with nvcc for sm_100a.

The shared object lands in ``nitrix_b200/_lib/`` next to the sources so that it
travels with a checkout (it is not installed into site-packages).  nvcc
cross-compiles without a GPU, so this runs on a CPU-only host as well.
"""
from __future__ import annotations

import hashlib
import os
import pathlib
import shutil
import subprocess

PKG = pathlib.Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
LIBDIR = PKG / "_lib"
LIBNAME = "libnitrix_b200_attention.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-shared", "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]


def sources() -> list[pathlib.Path]:
    return sorted(CSRC.glob("*.cu"))


def _digest() -> str:
    h = hashlib.sha256()
    for f in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def lib_path() -> pathlib.Path:
    return LIBDIR / LIBNAME


def is_current() -> bool:
    stamp = LIBDIR / "build.sha256"
    return lib_path().exists() and stamp.exists() and stamp.read_text().strip() == _digest()


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    """Compile every ``csrc/*.cu`` into one shared library (no-op when current)."""
    if not force and is_current():
        return lib_path()
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; cannot build " + LIBNAME)
    LIBDIR.mkdir(exist_ok=True)
    tmp = LIBDIR / (LIBNAME + ".tmp")
    cmd = [nvcc, *NVCC_FLAGS, f"-I{INCLUDE}", f"-I{CSRC}", "-o", str(tmp), *map(str, sources())]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stderr)
    os.replace(tmp, lib_path())
    (LIBDIR / "build.sha256").write_text(_digest() + "\n")
    return lib_path()


if __name__ == "__main__":
    import sys

    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
