"""Compile the reference project's own GPU kernels (legacy WMMA / mma.sync) for sm_100a.

TEST INFRASTRUCTURE: measurement and cross-check fixtures only -- never product code.  The kernel sources are compiled
where they lie in the reference checkout (nothing is copied) with the -D macros the reference's
host code passes to NVRTC (src/mma/GEMM.cpp:140-214, src/mma/Kernel*.cpp for the tile parameters).
Shapes are compile-time constants in those kernels, so there is one cubin per case; cubins and a
manifest go to oracle/_ref/gpu/ (git-ignored; carried to the GPU box like other built files).

    python oracle/build_reference_gpu.py
"""
from __future__ import annotations

import json
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref", "gpu")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
# checkout of the reference project: CCGLIB_REFERENCE_ROOT, else `reference` beside this repository
REF = os.environ.get("CCGLIB_REFERENCE_ROOT") or os.path.join(
    os.path.dirname(os.path.dirname(HERE)), "reference")

# ValueType ordinals (include/ccglib/common/value_type.h:14-22)
VT = {"int1": 0, "int32": 1, "bf16": 2, "e4m3": 3, "e5m2": 4, "f16": 5, "f32": 6}
BITS = {"int1": 1, "int32": 32, "bf16": 16, "e4m3": 8, "e5m2": 8, "f16": 16, "f32": 32}

# tile parameters per input type: m_blk, m_warp, m_wmma, n_blk, n_warp, n_wmma, k_wmma
TILES = {
    "f16": (128, 128, 16, 64, 16, 16, 16),
    "bf16": (128, 128, 16, 64, 16, 16, 16),
    "f32": (128, 128, 16, 64, 16, 16, 8),
    "e4m3": (128, 32, 16, 32, 32, 8, 32),
    "e5m2": (128, 32, 16, 32, 32, 8, 32),
    "int1": (64, 32, 16, 64, 32, 8, 256),
}

# name: (type_in, type_out, variant, B, M, N, K)
CASES = {
    "small_f16_basic": ("f16", "f32", "basic", 3, 128, 256, 64),
    "small_f16_opt": ("f16", "f32", "opt", 3, 128, 256, 64),
    "small_e4m3_opt": ("e4m3", "f32", "opt", 2, 128, 256, 128),
    "small_int1_opt": ("int1", "int32", "opt", 2, 128, 256, 512),
    "c1_f16_basic": ("f16", "f32", "basic", 1, 1024, 1024, 1024),
    "c2_f16_opt_b2": ("f16", "f32", "opt", 2, 8192, 8192, 8192),
    "c3_int1_opt_b1": ("int1", "int32", "opt", 1, 4096, 4096, 65536),
    "c4_e4m3_opt_b2": ("e4m3", "f32", "opt", 2, 4096, 4096, 16384),
    "c4_e5m2_opt_b2": ("e5m2", "f32", "opt", 2, 4096, 4096, 16384),
    "c5_bf16_basic_b64": ("bf16", "f32", "basic", 64, 256, 2048, 512),
    "c5_tf32_basic_b64": ("f32", "f32", "basic", 64, 256, 2048, 512),
}


def case_info(name: str) -> dict:
    tin, tout, variant, B, M, N, K = CASES[name]
    m_blk, m_warp, m_wmma, n_blk, n_warp, n_wmma, k_wmma = TILES[tin]
    block = (32, n_blk // n_warp, m_blk // m_warp)
    grid = (-(-N // n_blk), -(-M // m_blk), B)
    return {"name": name, "type_in": tin, "type_out": tout, "variant": variant, "B": B, "M": M,
            "N": N, "K": K, "m_blk": m_blk, "n_blk": n_blk, "k_chunk": k_wmma, "block": block,
            "grid": grid, "entry": "wmma_complex_gemm_" + variant,
            "cubin": name + ".cubin"}


def defines(info: dict) -> list[str]:
    tin, tout = info["type_in"], info["type_out"]
    m_blk, m_warp, m_wmma, n_blk, n_warp, n_wmma, k_wmma = TILES[tin]
    d = {
        "block_size_x": info["block"][0], "block_size_y": info["block"][1],
        "block_size_z": info["block"][2], "BATCH_SIZE": "%dUL" % info["B"],
        "M_GLOBAL": "%dUL" % info["M"], "N_GLOBAL": "%dUL" % info["N"],
        "K_GLOBAL": "%dUL" % info["K"], "K_PADDING": "0UL", "ALPHA_REAL": "1.000000",
        "ALPHA_IMAG": "0.000000", "BETA_REAL": "0.000000", "BETA_IMAG": "0.000000",
        "TYPE_IN": VT[tin], "TYPE_OUT": VT[tout], "NBIT_IN": BITS[tin], "NBIT_OUT": BITS[tout],
        "WARP_SIZE": 32, "M_PER_BLOCK": m_blk, "M_PER_WARP": m_warp, "M_PER_WMMA": m_wmma,
        "N_PER_BLOCK": n_blk, "N_PER_WARP": n_warp, "N_PER_WMMA": n_wmma, "K_PER_WMMA": k_wmma,
        "NBUFFER": 4,
    }
    flags = ["-D%s=%s" % kv for kv in d.items()]
    flags += ["-DC_COMPLEX_PLANAR", "-DA_ROW_MAJOR", "-DB_COL_MAJOR", "-DC_ROW_MAJOR"]
    return flags


def build(force: bool = False) -> str | None:
    kernels = os.path.join(REF, "kernels")
    if not os.path.isdir(kernels):
        return OUT if os.path.exists(os.path.join(OUT, "manifest.json")) else None
    os.makedirs(OUT, exist_ok=True)
    manifest = {}
    for name in CASES:
        info = case_info(name)
        src = os.path.join(kernels, "gemm_kernel_int1.cu" if info["type_in"] == "int1"
                           else "gemm_kernel_float.cu")
        cubin = os.path.join(OUT, info["cubin"])
        manifest[name] = info
        if not force and os.path.exists(cubin) and os.path.getmtime(cubin) >= max(
                os.path.getmtime(src), os.path.getmtime(__file__)):
            continue
        cmd = [os.path.join(CUDA_HOME, "bin", "nvcc"), "-std=c++17", "-arch=sm_100a", "-cubin",
               "-w", "-I", kernels, "-I", os.path.join(REF, "include"),
               "-I", os.path.join(REF, "include", "ccglib", "common"), "-o", cubin, src]
        cmd += defines(info)
        subprocess.run(cmd, check=True)
    with open(os.path.join(OUT, "manifest.json"), "w") as f:
        json.dump(manifest, f, indent=1)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
