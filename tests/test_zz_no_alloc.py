"""The allocation-free 1-bit GEMM entry point (scratch in a fixed array inside the library, for
callers that cannot call cudaMalloc once running) must give exactly what the plan-based entry
point gives.  Two calls in a row share the array; the second uses another shape so that anything
the first left behind would show.  This file sorts last on purpose: a run that stops at the first
failure has then already run every other test."""
import numpy as np
import pytest

import gpu_util as gu
import oracle_util as ou
from ccglib_b200 import capi

pytestmark = pytest.mark.gpu


def _inputs(seed, B, M, N, K):
    rng = np.random.default_rng(seed)
    kw = (K + 31) // 32
    a = ou.random_storage(rng, (B, 2, M, kw), ou.INT1)
    b = ou.random_storage(rng, (B, 2, N, kw), ou.INT1)
    pad = kw * 32 - K
    if pad:
        mask = np.uint32((1 << (32 - pad)) - 1)
        a[..., -1] &= mask
        b[..., -1] &= mask
    return a, b


def _run_static(a, b, B, M, N, K, **kw):
    import torch

    d_a, d_b = gu.dev(a), gu.dev(b)
    d_c = gu.dev_empty(B * 2 * M * N * 4, 0x5A)
    capi.gemm_int1_static_scratch(B, M, N, K, d_a.data_ptr(), d_b.data_ptr(), d_c.data_ptr(),
                                  gu.stream_handle(), **kw)
    torch.cuda.synchronize()
    gu.check_device_status()
    return gu.host(d_c, np.int32).copy()


def test_static_scratch_matches_plan_entry_point_twice_in_a_row():
    for seed, (B, M, N, K) in enumerate([(3, 200, 328, 2048), (2, 130, 72, 1000)]):
        a, b = _inputs(50 + seed, B, M, N, K)
        want = gu.run_gemm(ou.INT1, ou.INT32, a, b, B, M, N, K, variant=capi.BASIC)
        got = _run_static(a, b, B, M, N, K)
        assert np.array_equal(got, want)  # integer arithmetic: bit exact
        assert np.array_equal(got.reshape(B, 2, M, N),
                              gu.oracle_batch(ou.INT1, ou.INT32, a, b, B, M, N, K))


def test_static_scratch_batch_is_chunked_to_fit():
    # (3*256 + 2*512) * 8192 = 14 MiB per item: 5 items take three passes over the 32 MiB array
    B, M, N, K = 5, 256, 512, 8192
    a, b = _inputs(60, B, M, N, K)
    want = gu.run_gemm(ou.INT1, ou.INT32, a, b, B, M, N, K, variant=capi.BASIC)
    assert np.array_equal(_run_static(a, b, B, M, N, K), want)


def test_static_scratch_rejects_sizes_beyond_the_array():
    d = gu.dev_empty(256, 0)
    with pytest.raises(capi.Error) as err:
        capi.gemm_int1_static_scratch(1, 4096, 4096, 65536, d.data_ptr(), d.data_ptr(),
                                      d.data_ptr())
    assert err.value.status == capi.INVALID_ARGUMENT
    assert "built-in array holds" in str(err.value)
