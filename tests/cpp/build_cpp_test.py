"""Builds tests/cpp/bin/test_api: the C++ API (header-only, include/ccglib) exercised through the
stand-in cudawrappers header, linked against the CUDA library and the CPU oracle (as checker)."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
BIN = os.path.join(HERE, "bin", "test_api")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _load(name: str, path: str):
    import importlib.util

    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def build(force: bool = False) -> str:
    oracle_build = _load("oracle_build_recipe", os.path.join(ROOT, "oracle", "build.py"))
    lib_build = _load("ccglib_b200_build_recipe", os.path.join(ROOT, "ccglib_b200", "build.py"))

    lib = lib_build.build()
    port = oracle_build.build_port()
    src = os.path.join(HERE, "test_api.cpp")
    deps = [src, lib, port, os.path.join(ROOT, "include", "ccglib", "b200_api.hpp"),
            os.path.join(HERE, "shim", "cudawrappers", "cu.hpp"), __file__]
    if not force and os.path.exists(BIN) and all(
            os.path.getmtime(d) <= os.path.getmtime(BIN) for d in deps):
        return BIN
    os.makedirs(os.path.dirname(BIN), exist_ok=True)
    lib_dir, port_dir = os.path.dirname(lib), os.path.dirname(port)
    driver_dirs = [d for d in ("/usr/lib/x86_64-linux-gnu", os.path.join(CUDA_HOME, "lib64", "stubs"))
                   if os.path.exists(os.path.join(d, "libcuda.so"))]
    cmd = ["g++", "-std=c++17", "-O2", "-Wall", "-I", os.path.join(ROOT, "include"),
           "-I", os.path.join(HERE, "shim"), "-I", os.path.join(CUDA_HOME, "include"), src,
           "-o", BIN, "-L", lib_dir, "-lccglib_b200", "-L", port_dir, "-loracle_port",
           "-L", driver_dirs[0], "-lcuda", "-fopenmp",
           "-Wl,-rpath,$ORIGIN/" + os.path.relpath(lib_dir, os.path.dirname(BIN)),
           "-Wl,-rpath,$ORIGIN/" + os.path.relpath(port_dir, os.path.dirname(BIN))]
    subprocess.run(cmd, check=True)
    return BIN


REFERENCE_CLASS_LIB = os.path.join(HERE, "bin", "libreference_class.so")


def build_reference_class(force: bool = False) -> str:
    """C entry points (oracle/ref_wrap.cpp, the ones the tests already use for the reference's own
    CPU GEMM) compiled against THIS repository's include/ccglib/gemm/reference.h, so that the
    header-only ccglib::reference::GEMM can be called from Python.  Host only: no CUDA library."""
    wrap = os.path.join(ROOT, "oracle", "ref_wrap.cpp")
    header = os.path.join(ROOT, "include", "ccglib", "gemm", "reference.h")
    deps = [wrap, header, os.path.join(ROOT, "include", "ccglib", "b200_api.hpp"), __file__]
    if not force and os.path.exists(REFERENCE_CLASS_LIB) and all(
            os.path.getmtime(d) <= os.path.getmtime(REFERENCE_CLASS_LIB) for d in deps):
        return REFERENCE_CLASS_LIB
    os.makedirs(os.path.dirname(REFERENCE_CLASS_LIB), exist_ok=True)
    cmd = ["g++", "-std=c++17", "-O2", "-ffp-contract=off", "-fopenmp", "-fPIC", "-shared", "-Wall",
           "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA_HOME, "include"),
           "-o", REFERENCE_CLASS_LIB, wrap]
    subprocess.run(cmd, check=True)
    return REFERENCE_CLASS_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
    print(build_reference_class(force="--force" in sys.argv))
