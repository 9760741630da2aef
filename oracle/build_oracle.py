"""TEST INFRASTRUCTURE ONLY: builds the parity oracle's shared libraries.

* ``oracle/_build/libffi_oracle.so``  from ``oracle/ffi_oracle.c`` (gcc, OpenMP).
* ``oracle/_ref/libffi_ref.so``       the reference's own CPU kernels, compiled from
  ``tfsparse/cc/kernels/forward.cpp`` and ``backward.cpp`` where they lie in a checkout of
  the reference (path in ``$FFI_REFERENCE_ROOT``; a built-in default location is tried when it is unset), against
  the stand-in headers in ``oracle/ref_shim``.  Skipped when no checkout is present; a
  previously built library is then used as is.

Run ``python oracle/build_oracle.py`` or call :func:`build_all`.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "_build", "libffi_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libffi_ref.so")
# x86-64-v3 (AVX2+FMA) rather than -march=native: the library is built on one machine
# and run on another.
ARCH_FLAGS = ["-march=x86-64-v3"]


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_oracle(force: bool = False) -> str:
    src = os.path.join(HERE, "ffi_oracle.c")
    if not force and _newer(ORACLE_SO, [src]):
        return ORACLE_SO
    os.makedirs(os.path.dirname(ORACLE_SO), exist_ok=True)
    cmd = ["gcc", "-O3", "-std=c11", "-fPIC", "-shared", "-fopenmp", *ARCH_FLAGS, src, "-o", ORACLE_SO, "-lm"]
    subprocess.run(cmd, check=True)
    return ORACLE_SO


def reference_root() -> str:
    """Checkout of the reference: $FFI_REFERENCE_ROOT, else a `reference` directory beside this repository."""
    beside = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return os.environ.get("FFI_REFERENCE_ROOT", beside)


def build_reference(force: bool = False) -> str | None:
    """Compile the reference's CPU kernels; returns the path or None if unavailable."""
    kernels = os.path.join(reference_root(), "tfsparse", "cc", "kernels")
    sources = [os.path.join(kernels, "forward.cpp"), os.path.join(kernels, "backward.cpp")]
    adapter = os.path.join(HERE, "ref_adapter.cpp")
    if not all(os.path.exists(s) for s in sources):
        return REF_SO if os.path.exists(REF_SO) else None
    if not force and _newer(REF_SO, sources + [adapter]):
        return REF_SO
    os.makedirs(os.path.dirname(REF_SO), exist_ok=True)
    cmd = ["g++", "-std=c++17", "-O3", "-fPIC", "-shared", "-pthread", *ARCH_FLAGS,
           "-I", os.path.join(HERE, "ref_shim"), "-I", kernels, adapter, *sources, "-o", REF_SO]
    subprocess.run(cmd, check=True)
    return REF_SO


def build_all(force: bool = False) -> dict:
    return {"oracle": build_oracle(force), "reference": build_reference(force)}


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv))
