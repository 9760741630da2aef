"""Builds the CUDA library ``libffi_b200.so`` in-tree for sm_100a with nvcc.

``python -m ecml23_sparse_b200.build`` or :func:`build`.  The library is rebuilt when a
source file is newer than it.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")
INCLUDE = os.path.join(ROOT, "include")
LIB_PATH = os.path.join(PKG_DIR, "libffi_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=default",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the FFI library cannot be built")
    return exe


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(INCLUDE, "*.h"))
    return any(os.path.getmtime(d) > t for d in deps)


OBJ_DIR = os.path.join(PKG_DIR, "build")


def _compile_one(args) -> str:
    src, obj, extra, verbose = args
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", "-I", INCLUDE, "-I", CSRC, *extra, src, "-o", obj]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    return obj


def build(force: bool = False, verbose: bool = False, extra: list[str] | None = None) -> str:
    """Compiles every source file to an object (in parallel; an object is reused while it is newer than
    its source and the shared headers) and links them into the shared library."""
    if not force and not _stale():
        return LIB_PATH
    from concurrent.futures import ThreadPoolExecutor

    os.makedirs(OBJ_DIR, exist_ok=True)
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(INCLUDE, "*.h"))
    newest_header = max((os.path.getmtime(h) for h in headers), default=0.0)
    jobs, objs = [], []
    for src in sources():
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        fresh = (not force and not extra and os.path.exists(obj)
                 and os.path.getmtime(obj) > max(os.path.getmtime(src), newest_header))
        if not fresh:
            jobs.append((src, obj, extra or [], verbose))
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        list(pool.map(_compile_one, jobs))
    cmd = [_nvcc(), *NVCC_FLAGS, "-shared", *objs, "-o", LIB_PATH]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    return LIB_PATH


if __name__ == "__main__":
    extra = ["-Xptxas", "-v"] if "--ptxas" in sys.argv else None
    print(build(force=True, verbose=True, extra=extra))
