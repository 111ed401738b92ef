"""Ahead-of-time build of the CUDA library (sm_100a only) into ccglib_b200/lib/.

    python -m ccglib_b200.build [--force]
    python -m ccglib_b200.build --trace     # instrumented copy in ccglib_b200/lib/trace/

The shared library links the CUDA runtime statically and resolves the one driver entry point it
needs (cuTensorMapEncodeTiled) at run time, so it loads on machines without a GPU driver too.
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
OBJ_DIR = os.path.join(LIB_DIR, "obj")
LIB_PATH = os.path.join(LIB_DIR, "libccglib_b200.so")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")
SOURCES = ["gemm.cu", "pipeline.cu", "staging.cu", "transpose.cu", "packing.cu", "capi.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def _deps() -> list[str]:
    out = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    out.append(os.path.join(os.path.dirname(HERE), "include", "ccglib_b200.h"))
    out.append(__file__)
    return out


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _compile(src: str, verbose: bool) -> str:
    obj = os.path.join(OBJ_DIR, os.path.splitext(src)[0] + ".o")
    cmd = [NVCC] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + \
        ["-c", os.path.join(CSRC, src), "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s" % (src, res.stderr))
    if verbose:
        sys.stderr.write(res.stderr)
    return obj


def build_trace() -> str:
    """Instrumented copy of the library (-DCCGLIB_B200_TRACE: the GEMM kernel stamps the SM clock
    at tile start, last MMA issued, accumulator complete and epilogue done, see
    `python -m ccglib_b200.tune --timeline`).  Selected with CCGLIB_B200_LIB; never the default."""
    out_dir = os.path.join(LIB_DIR, "trace")
    obj_dir = os.path.join(out_dir, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    objs = []

    def one(src):
        obj = os.path.join(obj_dir, os.path.splitext(src)[0] + ".o")
        subprocess.run([NVCC] + NVCC_FLAGS + ["-DCCGLIB_B200_TRACE", "-c",
                                              os.path.join(CSRC, src), "-o", obj], check=True)
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        objs = list(pool.map(one, SOURCES))
    path = os.path.join(out_dir, "libccglib_b200.so")
    subprocess.run([NVCC, "-shared", "-o", path] + objs +
                   ["-gencode", "arch=compute_100a,code=sm_100a"], check=True)
    return path


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale(LIB_PATH, _deps()):
        return LIB_PATH
    os.makedirs(OBJ_DIR, exist_ok=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose), SOURCES))
    cmd = [NVCC, "-shared", "-o", LIB_PATH] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
    subprocess.run(cmd, check=True)
    return LIB_PATH


if __name__ == "__main__":
    if "--trace" in sys.argv:
        print(build_trace())
    else:
        print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
