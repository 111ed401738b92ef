"""Split-K form of the GEMM (a cluster of 2 or 4 CTAs shares the K of one 128 x 128 tile and
exchanges partial sums through distributed shared memory): chosen by the plan for problems that
leave most of the device idle, and forced here on ragged shapes, every floating-point kind, both
operand layouts and every C layout."""
import numpy as np
import pytest

import gpu_util as gu
import oracle_util as ou
from ccglib_b200 import capi
from test_gpu_gemm import make_inputs

pytestmark = pytest.mark.gpu


def test_plan_splits_k_for_a_single_small_problem():
    # BASELINE config 1: 64 tiles of 128 x 128 on 148 SMs -> two CTAs per tile
    plan = capi.GemmPlan(1, 1024, 1024, 1024, ou.F16, ou.F32, variant=capi.BASIC)
    assert plan.tile["split_k"] == 2 and plan.tile["bn"] == 128
    plan.close()
    plan = capi.GemmPlan(1, 512, 512, 4096, ou.F16, ou.F32, variant=capi.BASIC)
    assert plan.tile["split_k"] == 4  # 16 tiles
    plan.close()
    # enough tiles, 16-bit output or integer sums: no split
    for args in [(64, 1024, 1024, 1024, ou.F16, ou.F32), (1, 1024, 1024, 1024, ou.F16, ou.F16),
                 (1, 1024, 1024, 1024, ou.INT1, ou.INT32)]:
        plan = capi.GemmPlan(*args, variant=capi.BASIC)
        assert plan.tile["split_k"] == 1
        plan.close()


@pytest.mark.parametrize("split", [2, 4])
@pytest.mark.parametrize("types", [(ou.F16, ou.F32), (ou.BF16, ou.F32), (ou.F32, ou.F32),
                                   (ou.E4M3, ou.F32)], ids=["f16", "bf16", "tf32", "e4m3"])
def test_split_k_matches_float64_on_ragged_shapes(types, split, monkeypatch):
    monkeypatch.setenv("CCGLIB_B200_SPLITK", str(split))
    type_in, type_out = types
    # 3 x 5 tiles per item with ragged edges; 712 elements of K: k-blocks do not divide evenly
    B, M, N, K = 2, 300, 520, 712
    a, b = make_inputs(81, type_in, B, M, N, K, dist="uniform")
    for variant in (capi.BASIC, capi.OPT):
        plan = capi.GemmPlan(B, M, N, K, type_in, type_out, variant=variant)
        assert plan.tile["split_k"] == split
        plan.close()
        got = gu.run_gemm(type_in, type_out, a, b, B, M, N, K, variant=variant).reshape(B, 2, M, N)
        gu.assert_close_fp64(got, type_in, type_out, a, b, K)
        want = gu.oracle_batch(type_in, type_out, a, b, B, M, N, K)
        gu.assert_close_reference_rule(got, want, type_in, type_out)


@pytest.mark.parametrize("section", [(capi.PLANAR, capi.ROW_MAJOR), (capi.PLANAR, capi.COL_MAJOR),
                                     (capi.INTERLEAVED, capi.ROW_MAJOR),
                                     (capi.INTERLEAVED, capi.COL_MAJOR)],
                         ids=["planar-row", "planar-col", "inter-row", "inter-col"])
@pytest.mark.parametrize("split", [2, 4])
def test_split_k_every_c_layout_with_alpha_beta(section, split, monkeypatch):
    monkeypatch.setenv("CCGLIB_B200_SPLITK", str(split))
    c_axis, c_order = section
    B, M, N, K = 2, 200, 136, 1000
    alpha, beta = (0.5, 2.5), (0.25, -1.5)
    a, b = make_inputs(82, ou.F16, B, M, N, K, dist="uniform")
    rng = np.random.default_rng(83)
    c0 = rng.uniform(-1, 1, (B, 2, M, N)).astype(np.float32)  # canonical
    if c_axis == capi.PLANAR:
        c0_dev = c0.transpose(0, 1, 3, 2) if c_order == capi.COL_MAJOR else c0
    else:
        c0_dev = c0.transpose(0, 3, 2, 1) if c_order == capi.COL_MAJOR else c0.transpose(0, 2, 3, 1)
    got = gu.run_gemm(ou.F16, ou.F32, a, b, B, M, N, K, variant=capi.OPT, c_axis=c_axis,
                      c_order=c_order, alpha=alpha, beta=beta, c0=np.ascontiguousarray(c0_dev))
    got = gu.canonical_c(got, B, M, N, c_axis, c_order)
    want = gu.oracle_batch(ou.F16, ou.F32, a, b, B, M, N, K, alpha, beta, c0)
    gu.assert_close_reference_rule(got, want, ou.F16, ou.F32)
    assert np.allclose(got, want, rtol=2e-5, atol=4e-3)


def test_split_k_all_ones_and_determinism(monkeypatch):
    import torch

    monkeypatch.setenv("CCGLIB_B200_SPLITK", "4")
    B, M, N, K = 1, 256, 256, 2048
    ones = ou.quantize(np.ones((B, 2, M, K), np.float32), ou.F16)
    got = gu.run_gemm(ou.F16, ou.F32, ones, ones, B, M, N, K).reshape(B, 2, M, N)
    assert np.all(got[:, 0] == 0) and np.all(got[:, 1] == 2 * K)
    a, b = make_inputs(84, ou.F16, B, M, N, K, dist="uniform")
    d_a, d_b = gu.dev(a), gu.dev(b)
    plan = capi.GemmPlan(B, M, N, K, ou.F16, ou.F32, variant=capi.BASIC)
    outs = []
    for _ in range(3):
        d_c = gu.dev_empty(B * 2 * M * N * 4, 0xAB)
        plan.run(d_a.data_ptr(), d_b.data_ptr(), d_c.data_ptr(), gu.stream_handle())
        torch.cuda.synchronize()
        outs.append(d_c)
    gu.check_device_status()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    plan.close()
