"""ctypes access to the CPU oracle plus seeded input generators (test infrastructure).

Storage conventions (numpy side): float16 -> np.float16, bfloat16 -> np.uint16 bit
patterns, float8 e4m3/e5m2 -> np.uint8 bit patterns, float32 -> np.float32, 1-bit samples
-> np.uint32 words (sample i in bit i%32 of word i/32), int32 -> np.int32.
"""
from __future__ import annotations

import ctypes
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import build as oracle_build  # noqa: E402

# ValueType codes of the reference (include/ccglib/common/value_type.h:14-22)
INT1, INT32, BF16, E4M3, E5M2, F16, F32 = range(7)
TYPE_NAMES = {INT1: "int1", INT32: "int32", BF16: "bf16", E4M3: "e4m3", E5M2: "e5m2", F16: "f16",
              F32: "f32"}
STORAGE = {INT1: np.uint32, INT32: np.int32, BF16: np.uint16, E4M3: np.uint8, E5M2: np.uint8,
           F16: np.float16, F32: np.float32}
BITS = {INT1: 1, INT32: 32, BF16: 16, E4M3: 8, E5M2: 8, F16: 16, F32: 32}

_c_size_t = ctypes.c_size_t
_c_float = ctypes.c_float
_c_int = ctypes.c_int
_vp = ctypes.c_void_p


def _ptr(x: np.ndarray):
    assert x.flags["C_CONTIGUOUS"]
    return x.ctypes.data_as(_vp)


_port = None
_ref = False


def load_port():
    global _port
    if _port is None:
        path = oracle_build.build_port()
        lib = ctypes.CDLL(path)
        gemm_args = [_vp, _vp, _vp, _c_size_t, _c_size_t, _c_size_t, _c_int, _c_float, _c_float,
                     _c_float, _c_float]
        lib.oracle_cgemm_f32.argtypes = gemm_args
        lib.oracle_cgemm_f32.restype = None
        lib.oracle_cgemm_int1.argtypes = gemm_args
        lib.oracle_cgemm_int1.restype = None
        lib.oracle_widen.argtypes = [_vp, _vp, _c_size_t, _c_int]
        lib.oracle_widen.restype = _c_int
        lib.oracle_narrow.argtypes = [_vp, _vp, _c_size_t, _c_int]
        lib.oracle_narrow.restype = _c_int
        lib.oracle_pack_bits.argtypes = [_vp, _vp, _c_size_t, _c_int]
        lib.oracle_pack_bits.restype = None
        lib.oracle_unpack_bits.argtypes = [_vp, _vp, _c_size_t]
        lib.oracle_unpack_bits.restype = None
        lib.oracle_transpose.argtypes = [_vp, _vp] + [_c_size_t] * 6 + [_c_int]
        lib.oracle_transpose.restype = _c_int
        _port = lib
    return _port


def load_reference():
    """The reference project's own CPU GEMM, if it was (or can be) built; else None."""
    global _ref
    if _ref is False:
        try:
            path = oracle_build.build_reference()
        except Exception:
            path = None
        if path is None or not os.path.exists(path):
            _ref = None
        else:
            _ref = bind_reference_entry_points(ctypes.CDLL(path))
    return _ref


def bind_reference_entry_points(lib):
    """ctypes prototypes of the ten ref_gemm_* entry points of oracle/ref_wrap.cpp."""
    for name in ("e4m3_f32", "e5m2_f32", "f16_f16", "f16_f32", "f32_f16", "bf16_bf16",
                 "bf16_f32", "f32_bf16", "f32_f32", "int1_s32"):
        fn = getattr(lib, "ref_gemm_" + name)
        fn.argtypes = [_vp, _vp, _vp, _c_size_t, _c_size_t, _c_size_t, _c_int, _c_float,
                       _c_float, _c_float, _c_float]
        fn.restype = None
    return lib


# --------------------------------------------------------------------------- conversions

def widen(x: np.ndarray, value_type: int) -> np.ndarray:
    """Stored values -> float32 through the oracle's decoders."""
    x = np.ascontiguousarray(x)
    out = np.empty(x.shape, np.float32)
    rc = load_port().oracle_widen(_ptr(x), _ptr(out), x.size, value_type)
    assert rc == 0
    return out


def narrow(x: np.ndarray, value_type: int) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, STORAGE[value_type])
    rc = load_port().oracle_narrow(_ptr(x), _ptr(out), x.size, value_type)
    assert rc == 0
    return out


def to_double(x: np.ndarray, value_type: int) -> np.ndarray:
    if value_type == INT32:
        return x.astype(np.float64)
    return widen(x, value_type).astype(np.float64)


def quantize(x: np.ndarray, value_type: int) -> np.ndarray:
    """float32 values -> storage of value_type, round to nearest even."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    if value_type == F32:
        return x
    if value_type in (F16, BF16):
        return narrow(x, value_type)
    import torch

    dt = torch.float8_e4m3fn if value_type == E4M3 else torch.float8_e5m2
    return torch.from_numpy(x).to(dt).view(torch.uint8).numpy().copy()


def mask_tf32(x: np.ndarray) -> np.ndarray:
    """Clear the 13 low mantissa bits of float32 (what a tf32 tensor core consumes); the
    reference's tests prepare float32 inputs this way (test/gemm/mma.cpp:32-38)."""
    return (np.ascontiguousarray(x, np.float32).view(np.uint32) & np.uint32(0xFFFFE000)).view(
        np.float32)


# --------------------------------------------------------------------------- GEMM oracles

def port_gemm(type_in, type_out, a, b, c0, M, N, K, c_col_major=False, alpha=(1, 0), beta=(0, 0)):
    """One batch item through oracle.c.  a: [2][M][K'], b: [2][N][K'] storage arrays; c0: the
    previous C (storage of type_out) or None.  Returns C in storage of type_out, shape
    [2][M][N] or [2][N][M]."""
    lib = load_port()
    shape = (2, N, M) if c_col_major else (2, M, N)
    if type_in == INT1:
        c = np.zeros(shape, np.int32) if c0 is None else np.ascontiguousarray(c0, np.int32).copy()
        lib.oracle_cgemm_int1(_ptr(np.ascontiguousarray(a)), _ptr(np.ascontiguousarray(b)),
                              _ptr(c), M, N, K, int(c_col_major), alpha[0], alpha[1], beta[0],
                              beta[1])
        return c.reshape(shape)
    af = widen(a, type_in)
    bf = widen(b, type_in)
    cf = np.zeros(shape, np.float32) if c0 is None else widen(c0, type_out).reshape(shape)
    lib.oracle_cgemm_f32(_ptr(af), _ptr(bf), _ptr(cf), M, N, K, int(c_col_major), alpha[0],
                         alpha[1], beta[0], beta[1])
    return narrow(cf, type_out).reshape(shape)


def reference_gemm(ref, type_in, type_out, a, b, c0, M, N, K, c_col_major=False, alpha=(1, 0),
                   beta=(0, 0)):
    """Same contract as port_gemm but through the reference's own compiled CPU GEMM."""
    name = "ref_gemm_%s_%s" % (TYPE_NAMES[type_in], "s32" if type_out == INT32 else
                               TYPE_NAMES[type_out])
    fn = getattr(ref, name)
    shape = (2, N, M) if c_col_major else (2, M, N)
    c = (np.zeros(shape, STORAGE[type_out]) if c0 is None
         else np.ascontiguousarray(c0, STORAGE[type_out]).copy().reshape(shape))
    fn(_ptr(np.ascontiguousarray(a)), _ptr(np.ascontiguousarray(b)), _ptr(c), M, N, K,
       int(c_col_major), alpha[0], alpha[1], beta[0], beta[1])
    return c


def double_gemm(type_in, a, b, K=None):
    """float64 complex product of one batch item (row-major [2][M][N]) and the magnitude sums
    S_re = sum |ar||br| + |ai||bi|, S_im = sum |ar||bi| + |ai||br| used by the error bound."""
    if type_in == INT1:
        bits_a = np.unpackbits(np.ascontiguousarray(a).view(np.uint8), axis=-1, bitorder="little")
        bits_b = np.unpackbits(np.ascontiguousarray(b).view(np.uint8), axis=-1, bitorder="little")
        ad = bits_a[..., :K].astype(np.float64) * 2 - 1
        bd = bits_b[..., :K].astype(np.float64) * 2 - 1
    else:
        ad = widen(a, type_in).astype(np.float64)
        bd = widen(b, type_in).astype(np.float64)
    re = ad[0] @ bd[0].T - ad[1] @ bd[1].T
    im = ad[0] @ bd[1].T + ad[1] @ bd[0].T
    aa = np.abs(ad)
    ab = np.abs(bd)
    s_re = aa[0] @ ab[0].T + aa[1] @ ab[1].T
    s_im = aa[0] @ ab[1].T + aa[1] @ ab[0].T
    return np.stack([re, im]), np.stack([s_re, s_im])


# --------------------------------------------------------------------------- other oracles

def port_pack(bytes_in: np.ndarray, interleaved=False) -> np.ndarray:
    n = bytes_in.size
    out = np.zeros((n + 31) // 32, np.uint32)
    load_port().oracle_pack_bits(_ptr(np.ascontiguousarray(bytes_in, np.uint8)), _ptr(out), n,
                                 int(interleaved))
    return out


def port_unpack(words: np.ndarray, n: int) -> np.ndarray:
    out = np.zeros(n, np.uint8)
    load_port().oracle_unpack_bits(_ptr(np.ascontiguousarray(words, np.uint32)), _ptr(out), n)
    return out


def port_transpose(x: np.ndarray, B, M, N, Mc, Nc, nr_bits, interleaved=False) -> np.ndarray:
    """x: flat storage array of the whole input; returns the flat tiled output."""
    es = 4 if nr_bits == 1 else nr_bits // 8
    n_el = N // 32 if nr_bits == 1 else N
    nc_el = Nc // 32 if nr_bits == 1 else Nc
    mt = -(-M // Mc)
    nt = -(-n_el // nc_el)
    x = np.ascontiguousarray(x)
    assert x.nbytes == B * 2 * M * n_el * es
    out = np.zeros(B * mt * nt * 2 * Mc * nc_el * es, np.uint8)
    rc = load_port().oracle_transpose(_ptr(x), _ptr(out), B, M, N, Mc, Nc, nr_bits,
                                      int(interleaved))
    assert rc == 0
    return out.view(x.dtype)


# --------------------------------------------------------------------------- seeded inputs

def random_storage(rng: np.random.Generator, shape, value_type, dist="uniform", scale=1.0):
    """Seeded input values in storage form.  dist: 'uniform' U[-scale, scale], 'normal'
    N(0, scale^2), 'unit' U[0, 1) (the reference's test fixture range, test/gemm/mma.cpp:144-217),
    'bits' raw random bits (int1)."""
    if value_type == INT1:
        return rng.integers(0, 2**32, size=shape, dtype=np.uint32)
    if dist == "uniform":
        x = rng.uniform(-scale, scale, size=shape).astype(np.float32)
    elif dist == "normal":
        x = (rng.standard_normal(size=shape) * scale).astype(np.float32)
    elif dist == "unit":
        x = rng.random(size=shape, dtype=np.float32)
    else:
        raise ValueError(dist)
    if value_type == F32:
        return mask_tf32(x)
    return quantize(x, value_type)


# Small cases whose outputs from the reference's own CPU GEMM are stored in
# tests/golden/reference_cpu_outputs.npz (see tests/golden/make_golden.py).
GOLDEN_CPU_CASES = [
    dict(name="f16_f32_row", type_in=F16, type_out=F32, M=33, N=17, K=70, c_col_major=False,
         alpha=(1, 0), beta=(0, 0), seed=101),
    dict(name="f16_f32_col_ab", type_in=F16, type_out=F32, M=20, N=24, K=64, c_col_major=True,
         alpha=(0.3, 1.6), beta=(0.8, -1.1), seed=102),
    dict(name="f16_f16_row_ab", type_in=F16, type_out=F16, M=16, N=40, K=48, c_col_major=False,
         alpha=(0.5, 2.5), beta=(0.25, -1.5), seed=103),
    dict(name="bf16_f32_row", type_in=BF16, type_out=F32, M=24, N=16, K=96, c_col_major=False,
         alpha=(1, 0), beta=(0, 0), seed=104),
    dict(name="bf16_bf16_col", type_in=BF16, type_out=BF16, M=16, N=16, K=32, c_col_major=True,
         alpha=(1, 0), beta=(0, 0), seed=105),
    dict(name="f32_f32_row", type_in=F32, type_out=F32, M=19, N=23, K=40, c_col_major=False,
         alpha=(1, 0), beta=(0, 0), seed=106),
    dict(name="f32_f16_row", type_in=F32, type_out=F16, M=16, N=16, K=40, c_col_major=False,
         alpha=(1, 0), beta=(0, 0), seed=107),
    dict(name="f32_bf16_col_ab", type_in=F32, type_out=BF16, M=16, N=24, K=40, c_col_major=True,
         alpha=(2.0, -1.0), beta=(0.5, 0.5), seed=108),
    dict(name="e4m3_f32_row", type_in=E4M3, type_out=F32, M=32, N=16, K=64, c_col_major=False,
         alpha=(1, 0), beta=(0, 0), seed=109),
    dict(name="e5m2_f32_col", type_in=E5M2, type_out=F32, M=16, N=32, K=64, c_col_major=True,
         alpha=(1, 0), beta=(0, 0), seed=110),
    dict(name="int1_row", type_in=INT1, type_out=INT32, M=16, N=24, K=256, c_col_major=False,
         alpha=(1, 0), beta=(0, 0), seed=111),
    dict(name="int1_col_ab_padded", type_in=INT1, type_out=INT32, M=8, N=16, K=70,
         c_col_major=True, alpha=(2, 3), beta=(-1, 2), seed=112),
]


def golden_case_inputs(case):
    rng = np.random.default_rng(case["seed"])
    M, N, K = case["M"], case["N"], case["K"]
    if case["type_in"] == INT1:
        kw = (K + 31) // 32
        a = random_storage(rng, (2, M, kw), INT1)
        b = random_storage(rng, (2, N, kw), INT1)
        pad = kw * 32 - K
        if pad:  # padding bits are zero by contract (src/reference/GEMM.cpp:165-167)
            mask = np.uint32((1 << (32 - pad)) - 1)
            a[..., -1] &= mask
            b[..., -1] &= mask
        c0 = rng.integers(-50, 50, size=(2, M, N), dtype=np.int32)
    else:
        a = random_storage(rng, (2, M, K), case["type_in"], "uniform")
        b = random_storage(rng, (2, N, K), case["type_in"], "uniform")
        c0 = random_storage(rng, (2, M, N), case["type_out"], "uniform")
    if case["beta"] == (0, 0) and case["type_in"] != INT1:
        c0 = None
    return a, b, c0
