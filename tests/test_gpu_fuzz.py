"""Seeded random shapes through every layout the GEMM accepts: ragged M, N, K around the tile
edges of all kernel forms (64 / 128 / 256-column tiles, 256-row CTA pairs with 128 / 192 / 224
columns on the 1-bit path), batch sizes that do and do not fill the device, planar / interleaved
and row- / col-major C, alpha and beta.  1-bit results must be identical to the oracle; floating
point must agree with it under the reference's own acceptance rule (test/gemm/fpequals.h:38-53)."""
import numpy as np
import pytest

import gpu_util as gu
import oracle_util as ou
from ccglib_b200 import capi
from test_gpu_gemm import make_inputs

import os

pytestmark = pytest.mark.gpu
# cases per fuzz test; CCGLIB_B200_FUZZ_CASES raises it for a soak run
CASES = int(os.environ.get("CCGLIB_B200_FUZZ_CASES", "40"))

EDGES = [1, 7, 63, 64, 65, 127, 128, 129, 191, 192, 193, 223, 224, 225, 255, 256, 257, 300, 448,
         449, 511, 513, 640]


def _cases(seed, count, types):
    rng = np.random.default_rng(seed)
    out = []
    for i in range(count):
        type_in, type_out = types[int(rng.integers(len(types)))]
        M = int(rng.choice(EDGES))
        N = int(rng.choice(EDGES))
        if type_in == ou.INT1:
            K = int(rng.choice([32, 70, 256, 1000, 1056, 4128]))
        else:
            K = int(rng.choice([8, 40, 64, 100, 264, 520]))
        B = int(rng.choice([1, 2, 5]))
        variant = capi.OPT if rng.integers(2) else capi.BASIC
        if type_in == ou.INT1 and variant == capi.OPT:
            K = -(-K // 32) * 32  # the tiling pass moves whole 32-sample words
        c_axis = capi.INTERLEAVED if (variant == capi.OPT and rng.integers(2)) else capi.PLANAR
        c_order = capi.COL_MAJOR if rng.integers(2) else capi.ROW_MAJOR
        scaled = bool(rng.integers(3) == 0)
        out.append((i, type_in, type_out, B, M, N, K, variant, c_axis, c_order, scaled))
    return out


def _run(case):
    i, type_in, type_out, B, M, N, K, variant, c_axis, c_order, scaled = case
    a, b = make_inputs(1000 + i, type_in, B, M, N, K)
    alpha, beta, c0_canon, c0 = (1.0, 0.0), (0.0, 0.0), None, None
    if scaled:
        rng = np.random.default_rng(2000 + i)
        if type_in == ou.INT1:
            alpha, beta = (2.0, -1.0), (1.0, 3.0)
            c0_canon = rng.integers(-40, 40, size=(B, 2, M, N), dtype=np.int32)
        else:
            alpha, beta = (0.5, -1.25), (0.75, 0.5)
            c0_canon = ou.random_storage(rng, (B, 2, M, N), type_out, "uniform")
        # the caller's C in the requested layout
        if c_axis == capi.PLANAR:
            c0 = c0_canon if c_order == capi.ROW_MAJOR else c0_canon.transpose(0, 1, 3, 2)
        else:
            c0 = (c0_canon.transpose(0, 2, 3, 1) if c_order == capi.ROW_MAJOR
                  else c0_canon.transpose(0, 3, 2, 1))
        c0 = np.ascontiguousarray(c0)
    got = gu.run_gemm(type_in, type_out, a, b, B, M, N, K, variant=variant, c_axis=c_axis,
                      c_order=c_order, alpha=alpha, beta=beta, c0=c0)
    got = gu.canonical_c(got, B, M, N, c_axis, c_order)
    want = gu.oracle_batch(type_in, type_out, a, b, B, M, N, K, alpha, beta, c0_canon)
    return got, want, a, b


@pytest.mark.parametrize("case", _cases(17, CASES, [(ou.INT1, ou.INT32)]),
                         ids=lambda c: "i1-%d-B%d-%dx%dx%d" % (c[0], c[3], c[4], c[5], c[6]))
def test_int1_random_shapes_bit_exact(case):
    got, want, _, _ = _run(case)
    assert np.array_equal(got, want)


FLOATS = [(ou.F16, ou.F32), (ou.BF16, ou.F32), (ou.F32, ou.F32), (ou.E4M3, ou.F32),
          (ou.E5M2, ou.F32), (ou.F16, ou.F16), (ou.BF16, ou.BF16), (ou.F32, ou.F16)]


@pytest.mark.parametrize("case", _cases(23, CASES, FLOATS),
                         ids=lambda c: "%s-%d-B%d-%dx%dx%d" % (ou.TYPE_NAMES[c[1]], c[0], c[3],
                                                                c[4], c[5], c[6]))
def test_float_random_shapes_reference_rule(case):
    got, want, a, b = _run(case)
    gu.assert_close_reference_rule(got, want, case[1], case[2])
    if not case[-1]:  # alpha = 1, beta = 0: the library's own, much tighter, gate applies as well
        gu.assert_close_fp64(got, case[1], case[2], a, b, case[6])


def _pipeline_cases(seed, count):
    rng = np.random.default_rng(seed)
    out = []
    for i in range(count):
        one_bit = bool(rng.integers(2))
        M = int(rng.choice(EDGES))
        N = int(rng.choice(EDGES))
        K = int(rng.choice([16, 24, 40, 70, 256, 1000, 1056, 2080] if one_bit
                           else [8, 40, 64, 100, 264, 520, 1100]))
        B = int(rng.choice([1, 2, 3, 5]))
        in_axis = capi.INTERLEAVED if rng.integers(2) else capi.PLANAR
        out_axis = capi.INTERLEAVED if rng.integers(2) else capi.PLANAR
        c_order = capi.COL_MAJOR if rng.integers(2) else capi.ROW_MAJOR
        host = bool(rng.integers(2))
        slice_items = int(rng.integers(1, B + 1))
        out.append((i, one_bit, B, M, N, K, in_axis, out_axis, c_order, host, slice_items))
    return out


@pytest.mark.parametrize("case", _pipeline_cases(29, max(20, CASES // 2)),
                         ids=lambda c: "%s-%d-B%d-%dx%dx%d-%s" % ("i1" if c[1] else "f16", c[0], c[2],
                                                                 c[3], c[4], c[5],
                                                                 "host" if c[9] else "dev"))
def test_pipeline_random_shapes(case):
    """The Pipeline on seeded random shapes: 1-bit byte samples or f16, planar or interleaved
    input and output, row- or col-major C, device operands or host operands cut into slices."""
    import torch

    i, one_bit, B, M, N, K, in_axis, out_axis, c_order, host, slice_items = case
    rng = np.random.default_rng(3000 + i)
    if one_bit:
        a = rng.integers(0, 2, (B, 2, M, K)).astype(np.uint8) * rng.integers(1, 256, (B, 2, M, K)).astype(np.uint8)
        b = rng.integers(0, 2, (B, 2, N, K)).astype(np.uint8)
        kw = -(-K // 32)
        def packed(x, rows):
            padded = np.zeros((B, 2, rows, kw * 32), np.uint8)
            padded[..., :K] = x != 0
            return np.packbits(padded, axis=-1, bitorder="little").view(np.uint32).reshape(
                B, 2, rows, kw)
        want = gu.oracle_batch(ou.INT1, ou.INT32, packed(a, M), packed(b, N), B, M, N, K)
        tin, tout, out_dt = ou.INT1, ou.INT32, np.int32
    else:
        a = ou.random_storage(rng, (B, 2, M, K), ou.F16, "uniform")
        b = ou.random_storage(rng, (B, 2, N, K), ou.F16, "uniform")
        want = gu.oracle_batch(ou.F16, ou.F32, a, b, B, M, N, K)
        tin, tout, out_dt = ou.F16, ou.F32, np.float32
    a_in = np.ascontiguousarray(a.transpose(0, 2, 3, 1)) if in_axis == capi.INTERLEAVED else a
    b_in = np.ascontiguousarray(b.transpose(0, 2, 3, 1)) if in_axis == capi.INTERLEAVED else b
    pipe = capi.Pipeline(B, M, N, K, tin, tout, variant=capi.OPT, input_complex_axis=in_axis,
                         output_complex_axis=out_axis, c_mem_order=c_order)
    c_bytes = B * 2 * M * N * 4
    if host:
        pipe.host_slice = slice_items
        h_a, h_b = np.ascontiguousarray(a_in), np.ascontiguousarray(b_in)
        h_c = np.full(B * 2 * M * N, 0x5A5A5A5A, np.uint32)
        pipe.run_host(h_a.ctypes.data, h_b.ctypes.data, h_c.ctypes.data, gu.stream_handle())
        raw = h_c.view(out_dt)
    else:
        d_a, d_b = gu.dev(a_in), gu.dev(b_in)
        d_c = gu.dev_empty(c_bytes + 512, 0x5A)
        pipe.run(d_a.data_ptr(), d_b.data_ptr(), d_c.data_ptr() + 256, gu.stream_handle())
        torch.cuda.synchronize()
        whole = d_c.cpu().numpy()
        assert np.all(whole[:256] == 0x5A) and np.all(whole[256 + c_bytes:] == 0x5A)
        raw = whole[256:256 + c_bytes].view(out_dt)
    gu.check_device_status()
    pipe.close()
    got = gu.canonical_c(raw, B, M, N, out_axis, c_order)
    if one_bit:
        assert np.array_equal(got, want)
    else:
        gu.assert_close_reference_rule(got, want, tin, tout)
        gu.assert_close_fp64(got, tin, tout, a, b, K)
