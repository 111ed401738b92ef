"""Build recipe for the CPU oracle (test infrastructure, not product code).

Two shared libraries are produced:

* ``oracle/_port/liboracle_port.so`` -- ``oracle/oracle.c``, the CPU restatement
  of the reference algorithms (always buildable: plain C + OpenMP).
* ``oracle/_ref/libccglib_reference.so`` -- the reference project's own CPU GEMM
  (``src/reference/GEMM.cpp``) compiled unmodified from where it lies, together
  with ``oracle/ref_wrap.cpp`` (C entry points) and ``oracle/ref_shim`` (a stand-in
  for the N-d indexing helper of xtensor, which is not installed).  Only built
  when the reference checkout is present; the reference's own CMake build needs
  network access for its dependencies and is not used.

Run ``python oracle/build.py`` or call :func:`build_all`.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PORT_DIR = os.path.join(HERE, "_port")
REF_DIR = os.path.join(HERE, "_ref")
PORT_LIB = os.path.join(PORT_DIR, "liboracle_port.so")
REF_LIB = os.path.join(REF_DIR, "libccglib_reference.so")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def reference_root() -> str:
    """Checkout of the reference project: CCGLIB_REFERENCE_ROOT, else a `reference` directory
    beside this repository.  When neither exists the reference builds are skipped."""
    return os.environ.get("CCGLIB_REFERENCE_ROOT") or os.path.join(
        os.path.dirname(os.path.dirname(HERE)), "reference")


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources if os.path.exists(s))


def build_port(force: bool = False) -> str:
    src = os.path.join(HERE, "oracle.c")
    if not force and _newer(PORT_LIB, [src, __file__]):
        return PORT_LIB
    os.makedirs(PORT_DIR, exist_ok=True)
    cmd = ["gcc", "-std=c99", "-O2", "-ffp-contract=off", "-fopenmp", "-fPIC", "-shared",
           "-Wall", "-o", PORT_LIB, src]
    subprocess.run(cmd, check=True)
    return PORT_LIB


def build_reference(force: bool = False) -> str | None:
    """Compile the reference CPU GEMM from its own sources; None if they are absent."""
    root = reference_root()
    ref_src = os.path.join(root, "src", "reference", "GEMM.cpp")
    if not os.path.exists(ref_src):
        return REF_LIB if os.path.exists(REF_LIB) else None
    wrap = os.path.join(HERE, "ref_wrap.cpp")
    shim = os.path.join(HERE, "ref_shim")
    if not force and _newer(REF_LIB, [ref_src, wrap, os.path.join(shim, "xtensor", "xadapt.hpp"),
                                      __file__]):
        return REF_LIB
    if shutil.which("g++") is None:
        return None
    os.makedirs(REF_DIR, exist_ok=True)
    cmd = ["g++", "-std=c++17", "-O3", "-fopenmp", "-fPIC", "-shared", "-w",
           "-I", shim, "-I", os.path.join(root, "include"), "-I", os.path.join(CUDA_HOME, "include"),
           "-o", REF_LIB, ref_src, wrap]
    subprocess.run(cmd, check=True)
    return REF_LIB


def build_all(force: bool = False) -> dict:
    return {"port": build_port(force), "reference": build_reference(force)}


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv))
