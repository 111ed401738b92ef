"""GPU parity tests of Transpose and Packing through the C ABI: exact equality against the CPU
oracle, re-expressing test/transpose/transpose.cpp:37-46,113-146 and
test/packing/packing.cpp:22-204 of the reference, plus ragged shapes and the vector/scalar
kernel boundaries."""
import numpy as np
import pytest

import gpu_util as gu
import oracle_util as ou
from ccglib_b200 import capi

pytestmark = pytest.mark.gpu


def run_transpose(x, B, M, N, Mc, Nc, bits, axis):
    import torch

    d_in = gu.dev(x)
    es = 4 if bits == 1 else bits // 8
    n_el, nc_el = (N // 32, Nc // 32) if bits == 1 else (N, Nc)
    out_bytes = B * (-(-M // Mc)) * (-(-n_el // nc_el)) * 2 * Mc * nc_el * es
    d_out = gu.dev_empty(out_bytes + 512, 0x5A)
    capi.transpose(B, M, N, Mc, Nc, bits, axis, d_in.data_ptr(), d_out.data_ptr() + 256,
                   gu.stream_handle())
    torch.cuda.synchronize()
    raw = d_out.cpu().numpy()
    assert np.all(raw[:256] == 0x5A) and np.all(raw[256 + out_bytes:] == 0x5A)
    return raw[256:256 + out_bytes].view(x.dtype)


TRANSPOSE_CASES = [
    # (bits, B, M, N, Mc, Nc): the reference's case, the GEMM tile contract, ragged shapes
    (16, 2, 256, 128, 64, 64), (8, 2, 256, 128, 64, 64), (32, 2, 256, 128, 64, 64),
    (1, 2, 256, 128, 64, 64),
    (16, 3, 300, 200, 128, 64), (16, 3, 300, 200, 256, 64), (8, 2, 130, 300, 128, 128),
    (32, 2, 100, 72, 256, 32), (1, 2, 100, 2048, 128, 1024), (1, 2, 70, 96, 256, 1024),
    (16, 2, 100, 60, 128, 64),   # rows of 120 bytes: scalar kernel
    (8, 2, 33, 40, 16, 8),       # chunk rows of 8 bytes: scalar kernel
    (16, 1, 5, 7, 4, 3),
]


@pytest.mark.parametrize("axis", [capi.PLANAR, capi.INTERLEAVED], ids=["planar", "interleaved"])
@pytest.mark.parametrize("case", TRANSPOSE_CASES, ids=lambda c: "x".join(map(str, c)))
def test_transpose_matches_oracle(case, axis):
    bits, B, M, N, Mc, Nc = case
    rng = np.random.default_rng(31)
    dt = {1: np.uint32, 8: np.uint8, 16: np.uint16, 32: np.uint32}[bits]
    n_el = N // 32 if bits == 1 else N
    shape = (B, M, n_el, 2) if axis == capi.INTERLEAVED else (B, 2, M, n_el)
    x = rng.integers(1, np.iinfo(dt).max, size=shape, dtype=dt)
    got = run_transpose(x, B, M, N, Mc, Nc, bits, axis)
    want = ou.port_transpose(x.ravel(), B, M, N, Mc, Nc, bits, axis == capi.INTERLEAVED)
    assert np.array_equal(got, want)


def run_pack(x, n, direction, axis, out_dtype, out_count):
    import torch

    d_in = gu.dev(x)
    out_bytes = out_count * np.dtype(out_dtype).itemsize
    d_out = gu.dev_empty(out_bytes + 512, 0x5A)
    capi.pack(n, direction, axis, d_in.data_ptr(), d_out.data_ptr() + 256, gu.stream_handle())
    torch.cuda.synchronize()
    raw = d_out.cpu().numpy()
    assert np.all(raw[:256] == 0x5A) and np.all(raw[256 + out_bytes:] == 0x5A)
    return raw[256:256 + out_bytes].view(out_dtype)


@pytest.mark.parametrize("n", [2048, 32, 64, 4096 * 33, 2048 + 13, 7, 1 << 22])
def test_pack_planar(n):
    rng = np.random.default_rng(n)
    x = rng.integers(0, 2, n).astype(np.uint8)
    got = run_pack(x, n, capi.FORWARD, capi.PLANAR, np.uint32, (n + 31) // 32)
    assert np.array_equal(got, ou.port_pack(x))


def test_pack_treats_any_nonzero_byte_as_one():
    n = 4096
    rng = np.random.default_rng(5)
    x = rng.integers(0, 256, n).astype(np.uint8)
    x[rng.random(n) < 0.5] = 0
    got = run_pack(x, n, capi.FORWARD, capi.PLANAR, np.uint32, n // 32)
    assert np.array_equal(got, ou.port_pack(x))


@pytest.mark.parametrize("n", [2048, 64, 128 * 37, 2048 + 32, 70])
def test_pack_interleaved(n):
    rng = np.random.default_rng(n + 1)
    x = rng.integers(0, 2, n).astype(np.uint8)
    got = run_pack(x, n, capi.FORWARD, capi.INTERLEAVED, np.uint32, (n + 31) // 32)
    assert np.array_equal(got, ou.port_pack(x, interleaved=True))


@pytest.mark.parametrize("n", [2048, 32, 16, 2048 + 13, 5, 1 << 22])
def test_unpack(n):
    rng = np.random.default_rng(n + 2)
    w = rng.integers(0, 2**32, (n + 31) // 32, dtype=np.uint32)
    got = run_pack(w, n, capi.BACKWARD, capi.PLANAR, np.uint8, n)
    assert np.array_equal(got, ou.port_unpack(w, n))


def test_pack_unpack_round_trip():
    n = 1 << 20
    rng = np.random.default_rng(9)
    x = rng.integers(0, 2, n).astype(np.uint8)
    w = run_pack(x, n, capi.FORWARD, capi.PLANAR, np.uint32, n // 32)
    back = run_pack(w, n, capi.BACKWARD, capi.PLANAR, np.uint8, n)
    assert np.array_equal(back, x)


def test_unpack_interleaved_is_rejected():
    d = gu.dev_empty(256, 0)
    with pytest.raises(capi.Error) as err:
        capi.pack(64, capi.BACKWARD, capi.INTERLEAVED, d.data_ptr(), d.data_ptr(), 0)
    assert err.value.status == capi.UNSUPPORTED
    assert "complex-interleaved input is not supported in unpacking kernel" in str(err.value)


def test_pipeline_int1_pack_transpose_gemm():
    """pack -> transpose -> opt GEMM on unpacked 0/1 bytes, as the reference's Pipeline does for
    1-bit input (src/pipeline/Pipeline.cpp:108-126; test/pipeline/pipeline.cpp:88-187)."""
    import torch

    B, M, N, K = 2, 512, 512, 512
    rng = np.random.default_rng(41)
    a_bytes = rng.integers(0, 2, (B, 2, M, K)).astype(np.uint8)
    b_bytes = rng.integers(0, 2, (B, 2, N, K)).astype(np.uint8)
    stream = gu.stream_handle()
    d_a, d_b = gu.dev(a_bytes), gu.dev(b_bytes)
    p_a, p_b = gu.dev_empty(a_bytes.size // 8), gu.dev_empty(b_bytes.size // 8)
    capi.pack(a_bytes.size, capi.FORWARD, capi.PLANAR, d_a.data_ptr(), p_a.data_ptr(), stream)
    capi.pack(b_bytes.size, capi.FORWARD, capi.PLANAR, d_b.data_ptr(), p_b.data_ptr(), stream)
    torch.cuda.synchronize()
    a_words = gu.host(p_a, np.uint32).reshape(B, 2, M, K // 32)
    b_words = gu.host(p_b, np.uint32).reshape(B, 2, N, K // 32)
    got = gu.run_gemm(ou.INT1, ou.INT32, a_words, b_words, B, M, N, K, variant=capi.OPT)
    want = gu.oracle_batch(ou.INT1, ou.INT32, a_words, b_words, B, M, N, K)
    assert np.array_equal(got.reshape(B, 2, M, N), want)
    # and against plain +-1 arithmetic on the unpacked samples
    av = a_bytes[0].astype(np.int64) * 2 - 1
    bv = b_bytes[0].astype(np.int64) * 2 - 1
    re = av[0] @ bv[0].T - av[1] @ bv[1].T
    im = av[0] @ bv[1].T + av[1] @ bv[0].T
    assert np.array_equal(got.reshape(B, 2, M, N)[0], np.stack([re, im]))
