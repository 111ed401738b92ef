"""Helpers for the GPU parity tests: device buffers through torch (plumbing only), calls through
the C ABI (ccglib_b200.capi), comparison rules."""
from __future__ import annotations

import math

import numpy as np

import oracle_util as ou
from ccglib_b200 import capi

STORAGE = ou.STORAGE
U24 = 2.0 ** -24


def dev(x: np.ndarray):
    """numpy array -> flat uint8 torch tensor on cuda:0 holding the same bytes."""
    import torch

    flat = np.ascontiguousarray(x).reshape(-1).view(np.uint8)
    return torch.from_numpy(flat.copy()).cuda()


def dev_empty(nbytes: int, fill: int | None = None):
    import torch

    if fill is None:
        return torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    return torch.full((nbytes,), fill, dtype=torch.uint8, device="cuda")


def host(t, dtype) -> np.ndarray:
    return t.cpu().numpy().view(dtype)


def stream_handle() -> int:
    import torch

    return int(torch.cuda.current_stream().cuda_stream)


def check_device_status():
    word = capi.device_status()
    assert word == 0, "device status word 0x%x (bounded wait gave up)" % word


def tiled_nbytes(B, rows, K, type_in, blk, k_c):
    es_bits = ou.BITS[type_in]
    rt = -(-rows // blk)
    kt = -(-K // k_c)
    return B * rt * kt * 2 * blk * k_c * es_bits // 8


def run_gemm(type_in, type_out, a, b, B, M, N, K, *, variant=capi.BASIC, c_axis=capi.PLANAR,
             c_order=capi.ROW_MAJOR, alpha=(1.0, 0.0), beta=(0.0, 0.0), c0=None,
             in_axis=capi.PLANAR, canary=True):
    """a, b: storage arrays of the whole batch in the basic layout ([B][2][rows][K'], or
    [B][rows][K'][2] when in_axis is interleaved, which needs variant=OPT).  For OPT the inputs
    go through the library's transpose first, as in the reference's tests
    (test/gemm/mma.cpp:272-284).  Returns C as a flat storage array (layout as requested)."""
    import torch

    d_a, d_b = dev(a), dev(b)
    stream = stream_handle()
    if variant == capi.OPT:
        m_blk, n_blk, k_c = capi.gemm_dims(type_in, type_out, variant)
        bits = ou.BITS[type_in]
        t_a = dev_empty(tiled_nbytes(B, M, K, type_in, m_blk, k_c), 0xA5)
        t_b = dev_empty(tiled_nbytes(B, N, K, type_in, n_blk, k_c), 0xA5)
        capi.transpose(B, M, K, m_blk, k_c, bits, in_axis, d_a.data_ptr(), t_a.data_ptr(), stream)
        capi.transpose(B, N, K, n_blk, k_c, bits, in_axis, d_b.data_ptr(), t_b.data_ptr(), stream)
        d_a, d_b = t_a, t_b
    else:
        assert in_axis == capi.PLANAR
    out_dt = STORAGE[type_out]
    c_bytes = B * 2 * M * N * np.dtype(out_dt).itemsize
    pad = 256 if canary else 0
    d_c = dev_empty(c_bytes + 2 * pad, 0x5A)
    if c0 is not None:
        d_c[pad:pad + c_bytes] = dev(c0)
    plan = capi.GemmPlan(B, M, N, K, type_in, type_out, variant=variant, c_complex_axis=c_axis,
                         c_mem_order=c_order, alpha=alpha, beta=beta)
    plan.run(d_a.data_ptr(), d_b.data_ptr(), d_c.data_ptr() + pad, stream)
    torch.cuda.synchronize()
    check_device_status()
    plan.close()
    raw = d_c.cpu().numpy()
    if canary:
        assert np.all(raw[:pad] == 0x5A) and np.all(raw[pad + c_bytes:] == 0x5A), \
            "GEMM wrote outside the C buffer"
    return raw[pad:pad + c_bytes].view(out_dt).copy()


def canonical_c(c_flat, B, M, N, c_axis, c_order):
    """Any C layout -> [B][2][M][N]."""
    if c_axis == capi.PLANAR:
        if c_order == capi.ROW_MAJOR:
            return c_flat.reshape(B, 2, M, N)
        return c_flat.reshape(B, 2, N, M).transpose(0, 1, 3, 2)
    if c_order == capi.ROW_MAJOR:
        return c_flat.reshape(B, M, N, 2).transpose(0, 3, 1, 2)
    return c_flat.reshape(B, N, M, 2).transpose(0, 3, 2, 1)


def oracle_batch(type_in, type_out, a, b, B, M, N, K, alpha=(1, 0), beta=(0, 0), c0=None,
                 use_reference=False):
    """CPU oracle over the batch; a, b planar basic layout; c0 canonical row-major planar
    [B][2][M][N] or None.  Returns [B][2][M][N] storage array."""
    out = []
    ref = ou.load_reference() if use_reference else None
    for i in range(B):
        args = (type_in, type_out, a[i], b[i], None if c0 is None else c0[i], M, N, K, False,
                alpha, beta)
        out.append(ou.reference_gemm(ref, *args) if ref is not None else ou.port_gemm(*args))
    return np.stack(out)


def out_rounding_unit(type_out):
    return {ou.F32: 0.0, ou.INT32: 0.0, ou.F16: 2.0 ** -11, ou.BF16: 2.0 ** -8}[type_out]


# Gate on the accumulation error in units of sqrt(2K) * 2^-24 * S.  Measured on this library's
# kernels with zero-mean data: 0.02-0.1 for every input type (fp8 included: the f8f6f4 pipe
# accumulates in full fp32).
FP64_GATE_UNITS = 4.0
# Elements one MMA instruction reduces before it adds to the accumulator (32 bytes of K).
MMA_K = {ou.F16: 16, ou.BF16: 16, ou.F32: 8, ou.E4M3: 32, ou.E5M2: 32}


def fp64_tolerance(type_in, type_out, K, s, c64):
    """The library's stated tolerance per element (see assert_close_fp64)."""
    u_out = max(out_rounding_unit(type_out), U24)
    steps = 2.0 * K / MMA_K[type_in]
    return (FP64_GATE_UNITS * math.sqrt(2 * K) * U24 * s + steps * 2.0 * U24 * np.abs(c64) +
            2.0 * u_out * np.abs(c64) + 1e-30)


def assert_close_fp64(got, type_in, type_out, a, b, K):
    """Stated tolerance of this library for floating-point types, against a float64 product
    of the same stored inputs (alpha = 1, beta = 0):

        |c - c64| <= 4 sqrt(2K) 2^-24 S  +  (2K / k_mma) 2^-23 |c64|  +  2 u_out |c64|

    S = sum_k |ar||br| + |ai||bi| (imaginary part: |ar||bi| + |ai||br|).  Products of two
    f16 / bf16 / tf32 / fp8 values are exact in float32, so the only error is the float32
    accumulation of 2K terms in tensor-core order.  First term: rounding errors that add like a
    random walk.  Second term: the tensor core's adder truncates, so every MMA instruction (k_mma =
    16 / 8 / 32 elements for 16-bit / tf32 / fp8 input, 2K / k_mma instructions per output value)
    may lose up to one unit in the last place of the running sum, always in the same direction;
    on same-sign data, where the running sum grows to |c64|, that bias is what remains (measured:
    0.3-0.5 of this term), on zero-mean data it vanishes against the first term.  Third term: the
    final rounding (2^-24 for float32 output, 2^-11 f16, 2^-8 bf16).  A kernel that lost a few
    accumulator bits, or dropped one of the four real products, fails this gate.  The
    term-by-term worst case 2 (2K + 2) 2^-24 S is checked as well but can never bind.  Returns
    the observed error in units of sqrt(2K) * 2^-24 * S."""
    got64 = ou.to_double(got, type_out)
    worst = 0.0
    u_out = max(out_rounding_unit(type_out), U24)
    for i in range(got64.shape[0]):
        c64, s = ou.double_gemm(type_in, a[i], b[i])
        err = np.abs(got64[i] - c64)
        tol = fp64_tolerance(type_in, type_out, K, s, c64)
        bad = err > tol
        assert not bad.any(), "fp64 gate: %d elements off, worst err %g (tol %g)" % (
            int(bad.sum()), float(err[bad].max()), float(tol[bad].max()))
        assert not (err > 2.0 * (2 * K + 2) * U24 * s + 2.0 * u_out * np.abs(c64) + 1e-30).any()
        if type_out == ou.F32:
            worst = max(worst, float((err / (math.sqrt(2 * K) * U24 * s + 1e-30)).max()))
    return worst


REF_EPS = {ou.E4M3: 0.125, ou.E5M2: 0.25, ou.F16: 2.0 ** -10, ou.F32: 2.0 ** -10,
           ou.BF16: 2.0 ** -7}


def assert_close_reference_rule(got, want, type_in, type_out):
    """The reference's own acceptance rule (test/gemm/fpequals.h:38-53):
    |x - y| / (|x| + |y| + 1) <= 10 * eps(Tin), 100 * eps for outputs narrower than 32 bits."""
    x = ou.to_double(got, type_out)
    y = ou.to_double(want, type_out)
    factor = 100.0 if ou.BITS[type_out] < 32 else 10.0
    rel = np.abs(x - y) / (np.abs(x) + np.abs(y) + 1.0)
    assert rel.max() <= factor * REF_EPS[type_in], "reference rule: rel err %g" % rel.max()
