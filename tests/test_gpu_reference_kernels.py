"""Cross-check against the reference's own GPU path: its legacy WMMA / mma.sync kernels, compiled
unmodified for sm_100a (oracle/build_reference_gpu.py), run on the same seeded inputs as this
library.  1-bit results must be identical; floating-point results must agree within the
reference's own acceptance rule (test/gemm/fpequals.h:38-53) and each must satisfy the float64
gate.  The larger cases also time the legacy kernel, which gives the "reference kernel on B200"
column of the baseline table (written as reference_gpu_timings.json into the directory named by
CCGLIB_B200_TIMINGS_DIR, when that directory exists)."""
import json
import os

import numpy as np
import pytest

import gpu_util as gu
import oracle_util as ou
import reference_gpu as rg
from ccglib_b200 import capi

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TYPES = {"f16": ou.F16, "bf16": ou.BF16, "f32": ou.F32, "e4m3": ou.E4M3, "e5m2": ou.E5M2,
         "int1": ou.INT1, "int32": ou.INT32}
TIMINGS = {}


def _need_cubins():
    if not rg.available():
        pytest.skip("reference GPU kernels were not compiled (oracle/build_reference_gpu.py)")


def _device_inputs(info, seed):
    """Seeded inputs generated on the device in the basic layout, as torch tensors."""
    import torch

    B, M, N, K = info["B"], info["M"], info["N"], info["K"]
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    tin = info["type_in"]
    if tin == "int1":
        a = torch.randint(-2**31, 2**31 - 1, (B, 2, M, K // 32), dtype=torch.int32, device="cuda",
                          generator=g)
        b = torch.randint(-2**31, 2**31 - 1, (B, 2, N, K // 32), dtype=torch.int32, device="cuda",
                          generator=g)
        return a, b
    dt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32,
          "e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}[tin]

    def gen(rows):
        x = torch.rand((B, 2, rows, K), device="cuda", generator=g) * 2 - 1
        if tin == "f32":  # tf32 operands: clear the 13 low mantissa bits, as the reference's tests do
            x = (x.view(torch.int32) & -8192).view(torch.float32)
        return x.to(dt)

    return gen(M), gen(N)


def _tiled(x, B, rows, K, bits, blk, k_chunk):
    import torch

    rt, kt = -(-rows // blk), -(-K // k_chunk)
    out = torch.zeros(B * rt * kt * 2 * blk * k_chunk * bits // 8, dtype=torch.uint8, device="cuda")
    capi.transpose(B, rows, K, blk, k_chunk, bits, capi.PLANAR, x.data_ptr(), out.data_ptr(),
                   gu.stream_handle())
    return out


def _run_both(name, seed=5, time_it=False):
    import torch

    info = rg.manifest()[name]
    B, M, N, K = info["B"], info["M"], info["N"], info["K"]
    tin, tout = TYPES[info["type_in"]], TYPES[info["type_out"]]
    bits = ou.BITS[tin]
    a, b = _device_inputs(info, seed)
    stream = gu.stream_handle()
    out_dt = torch.int32 if tout == ou.INT32 else torch.float32
    # reference kernel (its own tile contract for the opt layout)
    if info["variant"] == "opt":
        ra = _tiled(a, B, M, K, bits, info["m_blk"], info["k_chunk"])
        rb = _tiled(b, B, N, K, bits, info["n_blk"], info["k_chunk"])
    else:
        ra, rb = a, b
    c_ref = torch.zeros((B, 2, M, N), dtype=out_dt, device="cuda")
    rg.launch(name, c_ref.data_ptr(), ra.data_ptr(), rb.data_ptr(), stream)
    torch.cuda.synchronize()
    # this library
    variant = capi.OPT if info["variant"] == "opt" else capi.BASIC
    if variant == capi.OPT:
        m_blk, n_blk, k_c = capi.gemm_dims(tin, tout, variant)
        oa = _tiled(a, B, M, K, bits, m_blk, k_c)
        ob = _tiled(b, B, N, K, bits, n_blk, k_c)
    else:
        oa, ob = a, b
    c_ours = torch.zeros((B, 2, M, N), dtype=out_dt, device="cuda")
    plan = capi.GemmPlan(B, M, N, K, tin, tout, variant=variant)
    plan.run(oa.data_ptr(), ob.data_ptr(), c_ours.data_ptr(), stream)
    torch.cuda.synchronize()
    gu.check_device_status()
    if time_it:
        def timed(fn, reps=3):
            fn()
            torch.cuda.synchronize()
            best = float("inf")
            for _ in range(reps):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                best = min(best, e0.elapsed_time(e1))
            return best

        ms_ref = timed(lambda: rg.launch(name, c_ref.data_ptr(), ra.data_ptr(), rb.data_ptr(),
                                         stream))
        ms_ours = timed(lambda: plan.run(oa.data_ptr(), ob.data_ptr(), c_ours.data_ptr(), stream))
        ops = 8.0 * B * M * N * K
        TIMINGS[name] = {"reference_kernel_ms": ms_ref, "reference_kernel_tops": ops / ms_ref / 1e9,
                         "ours_ms": ms_ours, "ours_tops": ops / ms_ours / 1e9,
                         "shape": [B, M, N, K], "types": [info["type_in"], info["type_out"]],
                         "variant": info["variant"]}
        print("%s: reference kernel %.3f ms (%.1f TOPS), this library %.3f ms (%.1f TOPS)" % (
            name, ms_ref, ops / ms_ref / 1e9, ms_ours, ops / ms_ours / 1e9))
        out_dir = os.environ.get("CCGLIB_B200_TIMINGS_DIR", "")  # unset: nothing is written
        if out_dir and os.path.isdir(out_dir):
            with open(os.path.join(out_dir, "reference_gpu_timings.json"), "w") as f:
                json.dump(TIMINGS, f, indent=1)
    plan.close()
    return info, a, b, c_ref, c_ours


@pytest.mark.parametrize("name", ["small_f16_basic", "small_f16_opt", "small_e4m3_opt"])
def test_small_float_cases_agree_with_reference_kernel(name):
    _need_cubins()
    info, a, b, c_ref, c_ours = _run_both(name)
    tin, tout = TYPES[info["type_in"]], TYPES[info["type_out"]]
    a_np = a.view(gu_torch_storage(tin)).cpu().numpy().view(ou.STORAGE[tin])
    b_np = b.view(gu_torch_storage(tin)).cpu().numpy().view(ou.STORAGE[tin])
    ref, ours = c_ref.cpu().numpy(), c_ours.cpu().numpy()
    gu.assert_close_reference_rule(ours, ref, tin, tout)
    gu.assert_close_fp64(ours, tin, tout, a_np, b_np, info["K"])
    gu.assert_close_fp64(ref, tin, tout, a_np, b_np, info["K"])


def gu_torch_storage(value_type):
    import torch

    return {ou.F16: torch.float16, ou.BF16: torch.int16, ou.F32: torch.float32,
            ou.E4M3: torch.uint8, ou.E5M2: torch.uint8, ou.INT1: torch.int32}[value_type]


def test_small_int1_case_is_identical_to_reference_kernel():
    import torch

    _need_cubins()
    info, a, b, c_ref, c_ours = _run_both("small_int1_opt")
    assert torch.equal(c_ref, c_ours)
    a_np = a.cpu().numpy().view(np.uint32)
    b_np = b.cpu().numpy().view(np.uint32)
    want = gu.oracle_batch(ou.INT1, ou.INT32, a_np, b_np, info["B"], info["M"], info["N"],
                           info["K"])
    assert np.array_equal(c_ours.cpu().numpy(), want)


BIG = ["c1_f16_basic", "c2_f16_opt_b2", "c4_e4m3_opt_b2", "c4_e5m2_opt_b2", "c5_bf16_basic_b64",
       "c5_tf32_basic_b64"]


@pytest.mark.parametrize("name", BIG)
def test_baseline_shapes_agree_with_reference_kernel_and_time_it(name):
    import torch

    _need_cubins()
    info, a, b, c_ref, c_ours = _run_both(name, time_it=True)
    eps = gu.REF_EPS[TYPES[info["type_in"]]]
    x, y = c_ours.double(), c_ref.double()
    rel = ((x - y).abs() / (x.abs() + y.abs() + 1.0)).max().item()
    assert rel <= 10.0 * eps, "reference rule against the reference GPU kernel: %g" % rel


def test_config3_int1_identical_to_reference_kernel_and_time_it():
    import torch

    _need_cubins()
    info, a, b, c_ref, c_ours = _run_both("c3_int1_opt_b1", time_it=True)
    assert torch.equal(c_ref, c_ours)
