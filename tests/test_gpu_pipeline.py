"""The Pipeline through the C ABI (ccglib_b200_pipeline_*): the caller's matrices in their natural
layout to C, from device operands and from host operands (batch slices double-buffered inside the
library).  Re-expresses the reference's pipeline tests (test/pipeline/pipeline.cpp:17-187: f16
planar / interleaved with alpha and beta on an unaligned shape; 1-bit input given as one byte
per sample) and adds the layouts and slice counts the library supports beyond them."""
import numpy as np
import pytest

import gpu_util as gu
import oracle_util as ou
from ccglib_b200 import capi

pytestmark = pytest.mark.gpu


def _bytes_inputs(seed, B, M, N, K, nonzero_is_one=False):
    rng = np.random.default_rng(seed)
    a = rng.integers(0, 2, (B, 2, M, K)).astype(np.uint8)
    b = rng.integers(0, 2, (B, 2, N, K)).astype(np.uint8)
    if nonzero_is_one:  # any non-zero byte is a +1 sample
        a = a * rng.integers(1, 256, a.shape).astype(np.uint8)
    return a, b


def _packed(x):
    """[B][2][rows][K] bytes -> [B][2][rows][ceil(K/32)] words, sample k in bit k%32."""
    B, _, rows, K = x.shape
    kw = -(-K // 32)
    padded = np.zeros((B, 2, rows, kw * 32), np.uint8)
    padded[..., :K] = x != 0
    return np.packbits(padded, axis=-1, bitorder="little").view(np.uint32).reshape(B, 2, rows, kw)


def _interleave(x):
    return np.ascontiguousarray(x.transpose(0, 2, 3, 1))


INT1_CASES = [
    # id, B, M, N, K, in axis, out axis, variant, env
    ("planar-aligned", 3, 128, 256, 1024, capi.PLANAR, capi.PLANAR, capi.OPT, {}),
    ("planar-ragged-k70", 2, 100, 60, 70, capi.PLANAR, capi.PLANAR, capi.BASIC, {}),
    ("planar-k-odd-bytes", 2, 130, 300, 1000, capi.PLANAR, capi.INTERLEAVED, capi.OPT, {}),
    ("interleaved-in", 3, 200, 136, 1056, capi.INTERLEAVED, capi.PLANAR, capi.OPT, {}),
    ("interleaved-in-out-k-ragged", 2, 65, 129, 1004, capi.INTERLEAVED, capi.INTERLEAVED,
     capi.BASIC, {}),
    ("i8-route-planar", 2, 300, 200, 2016, capi.PLANAR, capi.PLANAR, capi.OPT,
     dict(CCGLIB_B200_INT1_MXF4="0")),
    ("i8-route-interleaved", 2, 140, 72, 488, capi.INTERLEAVED, capi.PLANAR, capi.OPT,
     dict(CCGLIB_B200_INT1_MXF4="0")),
    ("three-nibble-planes", 2, 300, 260, 2048, capi.INTERLEAVED, capi.PLANAR, capi.OPT,
     dict(CCGLIB_B200_MXF4_NEGATE="0")),
    ("three-nibble-planes-planar-in", 2, 260, 300, 2064, capi.PLANAR, capi.INTERLEAVED, capi.BASIC,
     dict(CCGLIB_B200_MXF4_NEGATE="0")),
    ("single-cta-unaligned-base", 1, 100, 96, 48, capi.PLANAR, capi.PLANAR, capi.OPT,
     dict(CCGLIB_B200_PAIR="0")),
]


@pytest.mark.parametrize("case", INT1_CASES, ids=[c[0] for c in INT1_CASES])
def test_int1_pipeline_from_byte_samples_bit_exact(case, monkeypatch):
    import torch

    _, B, M, N, K, in_axis, out_axis, variant, env = case
    for key, value in env.items():
        monkeypatch.setenv(key, value)
    a, b = _bytes_inputs(51, B, M, N, K, nonzero_is_one=True)
    want = gu.oracle_batch(ou.INT1, ou.INT32, _packed(a), _packed(b), B, M, N, K)
    a_dev = gu.dev(_interleave(a) if in_axis == capi.INTERLEAVED else a)
    b_dev = gu.dev(_interleave(b) if in_axis == capi.INTERLEAVED else b)
    c_bytes = B * 2 * M * N * 4
    d_c = gu.dev_empty(c_bytes + 512, 0x5A)
    pipe = capi.Pipeline(B, M, N, K, ou.INT1, ou.INT32, variant=variant,
                         input_complex_axis=in_axis, output_complex_axis=out_axis)
    assert pipe.launches % 3 == 0  # expand A, expand B, GEMM per chunk: no pack, no transpose
    pipe.run(a_dev.data_ptr(), b_dev.data_ptr(), d_c.data_ptr() + 256, gu.stream_handle())
    torch.cuda.synchronize()
    gu.check_device_status()
    raw = d_c.cpu().numpy()
    assert np.all(raw[:256] == 0x5A) and np.all(raw[256 + c_bytes:] == 0x5A)
    got = gu.canonical_c(raw[256:256 + c_bytes].view(np.int32), B, M, N, out_axis, capi.ROW_MAJOR)
    assert np.array_equal(got, want)
    pipe.close()


@pytest.mark.parametrize("in_axis", [capi.PLANAR, capi.INTERLEAVED], ids=["planar", "interleaved"])
def test_f16_pipeline_device_operands(in_axis):
    # test/pipeline/pipeline.cpp:17-86: unaligned 300 x 200 x 100, alpha and beta set
    import torch

    B, M, N, K = 2, 300, 200, 100
    alpha, beta = (0.5, 2.0), (-1.5, 0.25)
    rng = np.random.default_rng(52)
    a = ou.random_storage(rng, (B, 2, M, K), ou.F16, "uniform")
    b = ou.random_storage(rng, (B, 2, N, K), ou.F16, "uniform")
    c0 = rng.uniform(-1, 1, (B, 2, M, N)).astype(np.float32)
    want = gu.oracle_batch(ou.F16, ou.F32, a, b, B, M, N, K, alpha, beta, c0)
    a_dev = gu.dev(_interleave(a) if in_axis == capi.INTERLEAVED else a)
    b_dev = gu.dev(_interleave(b) if in_axis == capi.INTERLEAVED else b)
    d_c = gu.dev(c0)
    pipe = capi.Pipeline(B, M, N, K, ou.F16, ou.F32, variant=capi.OPT, input_complex_axis=in_axis,
                         alpha=alpha, beta=beta)
    assert pipe.launches == 3  # transpose A, transpose B, GEMM
    pipe.run(a_dev.data_ptr(), b_dev.data_ptr(), d_c.data_ptr(), gu.stream_handle())
    torch.cuda.synchronize()
    gu.check_device_status()
    got = gu.host(d_c, np.float32).reshape(B, 2, M, N)
    gu.assert_close_reference_rule(got, want, ou.F16, ou.F32)
    assert np.allclose(got, want, rtol=2e-5, atol=2e-3)
    pipe.close()


@pytest.mark.parametrize("chunk", ["1", "2", "3"])
def test_f16_pipeline_chunks_overlap_transposes_and_gemm(chunk, monkeypatch):
    """With several chunks the transposes run on the pipeline's side stream beside the GEMM of
    earlier chunks; results are those of the single-chunk chain, call after call (the second call
    must not transpose into buffers the first call's GEMMs are still reading)."""
    import torch

    B, M, N, K = 7, 300, 264, 200
    rng = np.random.default_rng(55)
    a = ou.random_storage(rng, (B, 2, M, K), ou.F16, "uniform")
    b = ou.random_storage(rng, (B, 2, N, K), ou.F16, "uniform")
    a2 = ou.random_storage(rng, (B, 2, M, K), ou.F16, "uniform")
    d_a, d_b, d_a2 = gu.dev(_interleave(a)), gu.dev(_interleave(b)), gu.dev(_interleave(a2))
    monkeypatch.setenv("CCGLIB_B200_PIPE_CHUNK", chunk)
    pipe = capi.Pipeline(B, M, N, K, ou.F16, ou.F32, variant=capi.OPT,
                         input_complex_axis=capi.INTERLEAVED)
    chunks = -(-B // int(chunk))
    assert pipe.launches == 3 * chunks
    pipe.set_overlap(False)
    assert pipe.launches == 3
    pipe.set_overlap(True)
    d_c1 = gu.dev_empty(B * 2 * M * N * 4, 0xEE)
    d_c2 = gu.dev_empty(B * 2 * M * N * 4, 0xEE)
    side = torch.cuda.Stream()  # a non-blocking caller stream
    with torch.cuda.stream(side):
        pipe.run(d_a.data_ptr(), d_b.data_ptr(), d_c1.data_ptr(), int(side.cuda_stream))
        pipe.run(d_a2.data_ptr(), d_b.data_ptr(), d_c2.data_ptr(), int(side.cuda_stream))
    side.synchronize()  # only the caller's stream
    gu.check_device_status()
    for d_c, aa in ((d_c1, a), (d_c2, a2)):
        got = gu.host(d_c, np.float32).reshape(B, 2, M, N)
        gu.assert_close_fp64(got, ou.F16, ou.F32, aa, b, K)
    pipe.close()


def _pinned(x):
    import torch

    return torch.from_numpy(np.ascontiguousarray(x).reshape(-1).view(np.uint8).copy()).pin_memory()


@pytest.mark.parametrize("pinned", [True, False], ids=["pinned", "pageable"])
@pytest.mark.parametrize("slice_items", [1, 2, 5], ids=["slices-of-1", "slices-of-2", "one-slice"])
def test_host_operands_sliced_f16(slice_items, pinned):
    """Host A, B, C with beta != 0 (C is copied in as well), batch 5 cut into slices of 1, 2 (a
    short last slice) or everything at once: the result does not depend on the slicing."""
    B, M, N, K = 5, 260, 200, 136
    alpha, beta = (1.5, -0.5), (0.25, 1.0)
    rng = np.random.default_rng(53)
    a = ou.random_storage(rng, (B, 2, M, K), ou.F16, "uniform")
    b = ou.random_storage(rng, (B, 2, N, K), ou.F16, "uniform")
    c0 = rng.uniform(-1, 1, (B, 2, M, N)).astype(np.float32)
    want = gu.oracle_batch(ou.F16, ou.F32, a, b, B, M, N, K, alpha, beta, c0)
    pipe = capi.Pipeline(B, M, N, K, ou.F16, ou.F32, variant=capi.OPT,
                         input_complex_axis=capi.INTERLEAVED, alpha=alpha, beta=beta)
    pipe.host_slice = slice_items
    assert pipe.host_slice == slice_items
    if pinned:
        h_a, h_b, h_c = _pinned(_interleave(a)), _pinned(_interleave(b)), _pinned(c0)
        ptrs = (h_a.data_ptr(), h_b.data_ptr(), h_c.data_ptr())
    else:
        h_a, h_b = _interleave(a), _interleave(b)
        h_c = c0.copy()
        ptrs = (h_a.ctypes.data, h_b.ctypes.data, h_c.ctypes.data)
    pipe.run_host(*ptrs, gu.stream_handle())  # returns when C is complete in host memory
    got = (h_c.numpy().view(np.float32) if pinned else h_c).reshape(B, 2, M, N)
    gu.check_device_status()
    gu.assert_close_reference_rule(got, want, ou.F16, ou.F32)
    assert np.allclose(got, want, rtol=2e-5, atol=2e-3)
    with pytest.raises(capi.Error):  # the device slices exist now
        pipe.host_slice = 1
    # a second call reuses the slices and gives the same answer for beta = the same C input
    if pinned:
        h_c.copy_(_pinned(c0))
        pipe.run_host(*ptrs, gu.stream_handle())
        assert np.array_equal(h_c.numpy().view(np.float32).reshape(B, 2, M, N), got)
    pipe.close()


def test_host_operands_sliced_int1():
    # test/pipeline/pipeline.cpp:88-187 (bytes in host memory), here over three slices
    B, M, N, K = 6, 256, 128, 512
    a, b = _bytes_inputs(54, B, M, N, K)
    want = gu.oracle_batch(ou.INT1, ou.INT32, _packed(a), _packed(b), B, M, N, K)
    pipe = capi.Pipeline(B, M, N, K, ou.INT1, ou.INT32, variant=capi.OPT)
    pipe.host_slice = 2
    h_a, h_b = _pinned(a), _pinned(b)
    h_c = _pinned(np.zeros((B, 2, M, N), np.int32))
    pipe.run_host(h_a.data_ptr(), h_b.data_ptr(), h_c.data_ptr(), gu.stream_handle())
    gu.check_device_status()
    assert np.array_equal(h_c.numpy().view(np.int32).reshape(B, 2, M, N), want)
    pipe.close()


def test_pipeline_rejects_what_it_cannot_do():
    with pytest.raises(capi.Error) as err:  # nothing de-interleaves floats without the transpose
        capi.Pipeline(1, 64, 64, 64, ou.F16, ou.F32, variant=capi.BASIC,
                      input_complex_axis=capi.INTERLEAVED)
    assert err.value.status == capi.UNSUPPORTED
    with pytest.raises(capi.Error) as err:  # as the GEMM: basic variant writes planar C only
        capi.Pipeline(1, 64, 64, 64, ou.F16, ou.F32, variant=capi.BASIC,
                      output_complex_axis=capi.INTERLEAVED)
    assert err.value.status == capi.UNSUPPORTED
    with pytest.raises(capi.Error) as err:
        capi.Pipeline(1, 64, 64, 64, ou.INT1, ou.F32)
    assert err.value.status == capi.UNSUPPORTED
    pipe = capi.Pipeline(2, 64, 64, 64, ou.F16, ou.F32)
    with pytest.raises(capi.Error):
        pipe.host_slice = 3
    pipe.close()


def test_create_destroy_returns_all_device_memory():
    """Plans and pipelines own scratch, streams and events; creating, running and destroying
    them many times must leave the device's free memory where it was."""
    import torch

    B, M, N, K = 4, 256, 256, 512
    a, b = _bytes_inputs(56, B, M, N, K)
    d_a, d_b = gu.dev(a), gu.dev(b)
    d_c = gu.dev_empty(B * 2 * M * N * 4)
    h_c = np.zeros(B * 2 * M * N, np.int32)
    torch.cuda.synchronize()

    def cycle():
        pipe = capi.Pipeline(B, M, N, K, ou.INT1, ou.INT32)
        pipe.host_slice = 2
        pipe.run(d_a.data_ptr(), d_b.data_ptr(), d_c.data_ptr(), gu.stream_handle())
        pipe.run_host(a.ctypes.data, b.ctypes.data, h_c.ctypes.data, gu.stream_handle())
        pipe.close()
        fp = capi.Pipeline(B, M, N, K, ou.F16, ou.F32, input_complex_axis=capi.INTERLEAVED)
        fp.close()
        plan = capi.GemmPlan(B, M, N, K, ou.INT1, ou.INT32, variant=capi.BASIC)
        plan.close()

    cycle()  # first use loads modules and creates the context's pools
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for _ in range(25):
        cycle()
    torch.cuda.synchronize()
    free_after = torch.cuda.mem_get_info()[0]
    assert free_before - free_after < (8 << 20), "device memory leaked: %d bytes" % (
        free_before - free_after)
    gu.check_device_status()


@pytest.mark.parametrize("in_axis", [capi.PLANAR, capi.INTERLEAVED], ids=["planar", "interleaved"])
def test_int1_byte_samples_at_an_odd_address(in_axis):
    """Byte samples need no alignment: from an address that is not a multiple of 16 the front end
    reads sample by sample instead of in 16-byte pieces and gives the same result."""
    import torch

    B, M, N, K = 2, 72, 40, 1024
    a, b = _bytes_inputs(57, B, M, N, K)
    want = gu.oracle_batch(ou.INT1, ou.INT32, _packed(a), _packed(b), B, M, N, K)
    a_in = _interleave(a) if in_axis == capi.INTERLEAVED else a
    b_in = _interleave(b) if in_axis == capi.INTERLEAVED else b
    d_a = gu.dev_empty(a_in.size + 16, 0)
    d_b = gu.dev_empty(b_in.size + 16, 0)
    d_a[3:3 + a_in.size] = gu.dev(a_in)
    d_b[5:5 + b_in.size] = gu.dev(b_in)
    d_c = gu.dev_empty(B * 2 * M * N * 4, 0xEE)
    pipe = capi.Pipeline(B, M, N, K, ou.INT1, ou.INT32, input_complex_axis=in_axis)
    pipe.run(d_a.data_ptr() + 3, d_b.data_ptr() + 5, d_c.data_ptr(), gu.stream_handle())
    torch.cuda.synchronize()
    gu.check_device_status()
    pipe.close()
    assert np.array_equal(gu.host(d_c, np.int32).reshape(B, 2, M, N), want)


def test_misaligned_float_operands_are_rejected():
    """TMA needs 16-byte aligned operands; the GEMM says so instead of faulting."""
    d = gu.dev_empty(1 << 20, 0)
    plan = capi.GemmPlan(1, 128, 128, 128, ou.F16, ou.F32, variant=capi.BASIC)
    with pytest.raises(capi.Error) as err:
        plan.run(d.data_ptr() + 2, d.data_ptr(), d.data_ptr() + (1 << 19), gu.stream_handle())
    assert err.value.status == capi.INVALID_ARGUMENT and "16-byte aligned" in str(err.value)
    plan.close()
