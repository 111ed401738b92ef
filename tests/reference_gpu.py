"""TEST INFRASTRUCTURE: launches the reference project's own GPU kernels (compiled for sm_100a by
oracle/build_reference_gpu.py into oracle/_ref/gpu/) through the CUDA driver API, the way the
reference's host code does (kernel arguments (C, A, B); grid (ceil(N/n_blk), ceil(M/m_blk), B);
block (32, n_blk/n_warp, m_blk/m_warp); src/mma/GEMM.cpp:69-70,99-108, src/mma/Kernel.cpp:12-16).
Used only as a second checker and as the "legacy kernel on B200" baseline measurement."""
from __future__ import annotations

import ctypes
import json
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GPU_DIR = os.path.join(ROOT, "oracle", "_ref", "gpu")

_cuda = None
_modules = {}


def available() -> bool:
    return os.path.exists(os.path.join(GPU_DIR, "manifest.json"))


def manifest() -> dict:
    return json.load(open(os.path.join(GPU_DIR, "manifest.json")))


def _driver():
    global _cuda
    if _cuda is None:
        _cuda = ctypes.CDLL("libcuda.so.1")
    return _cuda


def _check(res, what):
    if res != 0:
        raise RuntimeError("%s failed with CUresult %d" % (what, res))


def kernel(name: str):
    """(CUfunction, case info) of one compiled case; needs a current CUDA context (torch)."""
    if name not in _modules:
        info = manifest()[name]
        drv = _driver()
        mod = ctypes.c_void_p()
        _check(drv.cuModuleLoad(ctypes.byref(mod), os.path.join(GPU_DIR, info["cubin"]).encode()),
               "cuModuleLoad")
        fn = ctypes.c_void_p()
        _check(drv.cuModuleGetFunction(ctypes.byref(fn), mod, info["entry"].encode()),
               "cuModuleGetFunction")
        _modules[name] = (fn, info, mod)
    return _modules[name][0], _modules[name][1]


def launch(name: str, d_c: int, d_a: int, d_b: int, stream: int) -> None:
    fn, info = kernel(name)
    args = [ctypes.c_uint64(d_c), ctypes.c_uint64(d_a), ctypes.c_uint64(d_b)]
    params = (ctypes.c_void_p * 3)(*[ctypes.cast(ctypes.byref(a), ctypes.c_void_p) for a in args])
    gx, gy, gz = info["grid"]
    bx, by, bz = info["block"]
    _check(_driver().cuLaunchKernel(fn, gx, gy, gz, bx, by, bz, 0, ctypes.c_void_p(stream), params,
                                    None), "cuLaunchKernel")
