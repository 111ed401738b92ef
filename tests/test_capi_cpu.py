"""CPU-only checks of the C-ABI library: it loads without a GPU driver, exports every symbol the
header declares, and validates arguments before touching CUDA."""
import os
import re

import pytest

from ccglib_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "ccglib_b200.h")).read()
    declared = sorted(set(re.findall(r"CCGLIB_B200_API[^;(]*?\b(ccglib_b200_[a-z0-9_]+)\s*\(", header)))
    assert declared == sorted(capi.EXPORTS)
    lib = capi.lib()
    for name in declared:
        assert getattr(lib, name) is not None


def test_gemm_dims_tile_contract():
    # one slab row is 128 bytes for every input type
    assert capi.gemm_dims(capi.FLOAT16) == (128, 256, 64)
    assert capi.gemm_dims(capi.BFLOAT16) == (128, 256, 64)
    assert capi.gemm_dims(capi.FLOAT32) == (128, 256, 32)
    assert capi.gemm_dims(capi.FLOAT8E4M3) == (128, 256, 128)
    assert capi.gemm_dims(capi.FLOAT8E5M2) == (128, 256, 128)
    assert capi.gemm_dims(capi.INT1, capi.INT32) == (128, 256, 1024)
    with pytest.raises(capi.Error):
        capi.gemm_dims(capi.INT32)
    with pytest.raises(capi.Error):
        capi.gemm_dims(42)


def test_plan_rejects_what_the_reference_rejects():
    # basic + interleaved C (src/mma/GEMM.cpp:77-80)
    with pytest.raises(capi.Error) as err:
        capi.GemmPlan(1, 128, 128, 128, capi.FLOAT16, capi.FLOAT32, variant=capi.BASIC,
                      c_complex_axis=capi.INTERLEAVED)
    assert err.value.status == capi.UNSUPPORTED
    assert "complex-interleaved output is not supported in basic variant" in str(err.value)
    # col-major A / row-major B (kernels/gemm_kernel_float.cu:20-25; test/gemm/mma.cpp:598-643)
    with pytest.raises(capi.Error) as err:
        capi.GemmPlan(1, 128, 128, 128, capi.FLOAT16, capi.FLOAT32, a_mem_order=capi.COL_MAJOR)
    assert err.value.status == capi.UNSUPPORTED and "col-major A" in str(err.value)
    with pytest.raises(capi.Error) as err:
        capi.GemmPlan(1, 128, 128, 128, capi.FLOAT16, capi.FLOAT32, b_mem_order=capi.ROW_MAJOR)
    assert err.value.status == capi.UNSUPPORTED and "row-major B" in str(err.value)


def test_plan_rejects_bad_sizes():
    for dims in [(0, 1, 1, 1), (1, 0, 1, 1), (1, 1, 0, 1), (1, 1, 1, 0)]:
        with pytest.raises(capi.Error) as err:
            capi.GemmPlan(*dims, capi.FLOAT16, capi.FLOAT32)
        assert err.value.status == capi.INVALID_ARGUMENT


def test_transpose_and_pack_validate_arguments():
    with pytest.raises(capi.Error) as err:
        capi.transpose(1, 8, 8, 4, 4, 16, capi.PLANAR, 0, 0)
    assert err.value.status == capi.INVALID_ARGUMENT
    with pytest.raises(capi.Error) as err:
        capi.transpose(1, 8, 8, 4, 4, 12, capi.PLANAR, 256, 512)
    assert err.value.status == capi.INVALID_ARGUMENT
    with pytest.raises(capi.Error) as err:
        capi.transpose(1, 8, 40, 4, 32, 1, capi.PLANAR, 256, 512)  # N not a multiple of 32
    assert err.value.status == capi.INVALID_ARGUMENT
    with pytest.raises(capi.Error) as err:
        capi.pack(0, capi.FORWARD, capi.PLANAR, 256, 512)
    assert err.value.status == capi.INVALID_ARGUMENT
    with pytest.raises(capi.Error) as err:
        capi.pack(64, capi.BACKWARD, capi.INTERLEAVED, 256, 512)
    assert err.value.status == capi.UNSUPPORTED
    with pytest.raises(capi.Error) as err:
        capi.pack(64, 7, capi.PLANAR, 256, 512)
    assert err.value.status == capi.INVALID_ARGUMENT


def test_status_strings():
    lib = capi.lib()
    assert lib.ccglib_b200_status_string(0) == b"success"
    assert lib.ccglib_b200_status_string(4) == b"device-side wait timed out"
