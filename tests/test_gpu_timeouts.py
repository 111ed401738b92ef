"""The bounded device-side waits of the GEMM kernels, made to run out without any fault: a wait on
a barrier nobody arrives on (host-made failure), with a limit of a fraction of a millisecond.
The kernel must return, the status word must say which wait gave up, the abort must reach the
other waiter (another warp, or the other CTA of a pair) long before its own limit, the status
must read clean afterwards, and the next GEMM must be correct."""
import numpy as np
import pytest

import gpu_util as gu
import oracle_util as ou
from ccglib_b200 import capi

pytestmark = pytest.mark.gpu

PRODUCER_BIT, EPILOGUE_BIT = 1, 4


@pytest.mark.parametrize("pair", [False, True], ids=["one-cta", "cta-pair"])
def test_wait_runs_out_and_status_reports_it(pair):
    import torch

    torch.cuda.synchronize()
    assert capi.device_status() == 0
    limit = 200_000  # about 0.1 ms of SM clock
    first, second = capi.selftest_wait_timeout(limit, pair)
    assert first >= limit  # the first waiter sat out its limit ...
    assert first < 50 * limit
    assert second < 50 * limit  # ... the second left through the abort flag, not its 200x limit
    word = ctypes_status()
    assert word == (capi.DEVICE_TIMEOUT, PRODUCER_BIT)  # only the first waiter's code
    assert capi.device_status() == 0  # sticky word is cleared by the read
    # the context is intact: a GEMM afterwards is correct and leaves the word clean
    B, M, N, K = 2, 300, 200, 136
    rng = np.random.default_rng(5)
    a = ou.random_storage(rng, (B, 2, M, K), ou.F16, "uniform")
    b = ou.random_storage(rng, (B, 2, N, K), ou.F16, "uniform")
    got = gu.run_gemm(ou.F16, ou.F32, a, b, B, M, N, K).reshape(B, 2, M, N)
    gu.assert_close_fp64(got, ou.F16, ou.F32, a, b, K)


def ctypes_status():
    import ctypes

    word = ctypes.c_uint(0)
    status = capi.lib().ccglib_b200_device_status(ctypes.byref(word))
    return status, int(word.value)


def test_selftest_rejects_unbounded_limits():
    with pytest.raises(capi.Error):
        capi.selftest_wait_timeout(0)
    with pytest.raises(capi.Error):
        capi.selftest_wait_timeout(10 ** 9)


def test_wait_limit_is_a_plan_parameter(monkeypatch):
    """CCGLIB_B200_WAIT_CYCLES sets the limit of a plan's kernels; a generous value changes
    nothing about the result."""
    monkeypatch.setenv("CCGLIB_B200_WAIT_CYCLES", "500000000")
    B, M, N, K = 1, 256, 256, 512
    rng = np.random.default_rng(6)
    a = ou.random_storage(rng, (B, 2, M, K // 32), ou.INT1)
    b = ou.random_storage(rng, (B, 2, N, K // 32), ou.INT1)
    got = gu.run_gemm(ou.INT1, ou.INT32, a, b, B, M, N, K).reshape(B, 2, M, N)
    assert np.array_equal(got, gu.oracle_batch(ou.INT1, ou.INT32, a, b, B, M, N, K))
