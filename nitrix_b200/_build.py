"""Builds the CUDA library in-tree with nvcc for sm_100a.

The shared object lands in ``nitrix_b200/_lib/`` next to the sources so that it
travels with a checkout (it is not installed into site-packages).  nvcc
cross-compiles without a GPU, so this runs on a CPU-only host as well.

Every ``csrc/*.cu`` is compiled to its own object file (in parallel, and only
when the file, a header or the flags changed since its object was made); the
objects are then linked into one shared library.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import pathlib
import shutil
import subprocess

PKG = pathlib.Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
LIBDIR = PKG / "_lib"
OBJDIR = LIBDIR / "obj"
LIBNAME = "libnitrix_b200_attention.so"

COMPILE_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]
LINK_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC"]


def sources() -> list[pathlib.Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers_digest() -> bytes:
    h = hashlib.sha256()
    for f in sorted(list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(COMPILE_FLAGS).encode())
    return h.digest()


def _object_digest(src: pathlib.Path, headers: bytes) -> str:
    h = hashlib.sha256(headers)
    h.update(src.name.encode())
    h.update(src.read_bytes())
    return h.hexdigest()


def _digest() -> str:
    headers = _headers_digest()
    h = hashlib.sha256()
    for f in sources():
        h.update(_object_digest(f, headers).encode())
    h.update(" ".join(LINK_FLAGS).encode())
    return h.hexdigest()


def lib_path() -> pathlib.Path:
    return LIBDIR / LIBNAME


def is_current() -> bool:
    stamp = LIBDIR / "build.sha256"
    return lib_path().exists() and stamp.exists() and stamp.read_text().strip() == _digest()


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; cannot build " + LIBNAME)
    return nvcc


def _compile_one(nvcc: str, src: pathlib.Path, obj: pathlib.Path, verbose: bool) -> str:
    cmd = [nvcc, *COMPILE_FLAGS, f"-I{INCLUDE}", f"-I{CSRC}", "-c", "-o", str(obj), str(src)]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    return res.stderr


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    """Compile every ``csrc/*.cu`` and link one shared library (no-op when current)."""
    if not force and not verbose and is_current():
        return lib_path()
    nvcc = _nvcc()
    OBJDIR.mkdir(parents=True, exist_ok=True)
    headers = _headers_digest()
    jobs = []
    objs = []
    for src in sources():
        obj = OBJDIR / (src.stem + ".o")
        stamp = OBJDIR / (src.stem + ".sha256")
        want = _object_digest(src, headers)
        objs.append(obj)
        if force or verbose or not obj.exists() or not stamp.exists() or stamp.read_text().strip() != want:
            jobs.append((src, obj, stamp, want))
    with concurrent.futures.ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 1))) as pool:
        futures = {pool.submit(_compile_one, nvcc, src, obj, verbose): (src, stamp, want) for src, obj, stamp, want in jobs}
        for fut in concurrent.futures.as_completed(futures):
            src, stamp, want = futures[fut]
            log = fut.result()
            stamp.write_text(want + "\n")
            if verbose:
                print(f"==== {src.name}\n{log}")
    tmp = LIBDIR / (LIBNAME + ".tmp")
    cmd = [nvcc, *LINK_FLAGS, "-o", str(tmp), *map(str, objs)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc link failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    os.replace(tmp, lib_path())
    (LIBDIR / "build.sha256").write_text(_digest() + "\n")
    return lib_path()


if __name__ == "__main__":
    import sys

    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
