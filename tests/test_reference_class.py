"""The header-only ccglib::reference::GEMM of this repository (include/ccglib/gemm/reference.h)
against what the reference's own class produces: its known-answer vectors
(test/gemm/reference.cpp, read into tests/golden/reference_test_vectors.json), stored outputs of
the reference's compiled CPU GEMM on seeded inputs, and -- where that GEMM could be compiled on
this machine -- the binary itself.  Host only."""
import ctypes
import json
import os
import sys

import numpy as np
import pytest

import oracle_util as ou

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")
VECTORS = json.load(open(os.path.join(GOLDEN, "reference_test_vectors.json")))
NAME_TO_TYPE = {"float16": ou.F16, "bfloat16": ou.BF16, "float32": ou.F32}


@pytest.fixture(scope="module")
def cls():
    sys.path.insert(0, os.path.join(ROOT, "tests", "cpp"))
    import build_cpp_test as cpp_build

    return ou.bind_reference_entry_points(ctypes.CDLL(cpp_build.build_reference_class()))


@pytest.mark.parametrize("type_name", VECTORS["float"]["input_types"])
@pytest.mark.parametrize("col", [False, True])
def test_float_known_answer(cls, type_name, col):
    v = VECTORS["float"]
    t = NAME_TO_TYPE[type_name]
    M, N, K = v["M"], v["N"], v["K"]
    a = ou.quantize(np.array(v["a"], np.float32).reshape(2, M, K), t)
    b = ou.quantize(np.array(v["b"], np.float32).reshape(2, N, K), t)
    c = ou.reference_gemm(cls, t, ou.F32, a, b, None, M, N, K, c_col_major=col)
    want = np.array(v["c_col_major" if col else "c_row_major"], np.float32)
    assert np.array_equal(c.ravel(), want)


@pytest.mark.parametrize("col", [False, True])
def test_binary_known_answer(cls, col):
    v = VECTORS["binary"]
    M, N, K = v["M"], v["N"], v["K"]
    a = np.array(v["a"], np.uint32).reshape(2, M, K // 32)
    b = np.array(v["b"], np.uint32).reshape(2, N, K // 32)
    c = ou.reference_gemm(cls, ou.INT1, ou.INT32, a, b, None, M, N, K, c_col_major=col)
    assert c.ravel().tolist() == v["c_col_major" if col else "c_row_major"]


def test_alpha_beta_known_answers(cls):
    v = VECTORS["alpha_beta_float16"]
    M, N, K = v["M"], v["N"], v["K"]
    a = ou.quantize(np.array(v["a"], np.float32).reshape(2, M, K), ou.F16)
    b = ou.quantize(np.array(v["b"], np.float32).reshape(2, N, K), ou.F16)
    c0 = np.array(v["c_in"], np.float32).reshape(2, M, N)
    c = ou.reference_gemm(cls, ou.F16, ou.F32, a, b, c0, M, N, K, alpha=tuple(v["alpha"]),
                          beta=tuple(v["beta"]))
    assert np.array_equal(c.ravel(), np.array(v["c_ref"], np.float32))
    v = VECTORS["alpha_beta_int1"]
    M, N, K = v["M"], v["N"], v["K"]
    a = np.array(v["a"], np.uint32).reshape(2, M, K // 32)
    b = np.array(v["b"], np.uint32).reshape(2, N, K // 32)
    c0 = np.array(v["c_in"], np.int32).reshape(2, M, N)
    c = ou.reference_gemm(cls, ou.INT1, ou.INT32, a, b, c0, M, N, K, alpha=tuple(v["alpha"]),
                          beta=tuple(v["beta"]))
    assert c.ravel().tolist() == v["c_ref"]


@pytest.mark.parametrize("case", ou.GOLDEN_CPU_CASES, ids=lambda c: c["name"])
def test_matches_stored_reference_outputs(cls, case):
    """All ten Run() overloads, row- and col-major, with and without alpha/beta: bit-identical to
    the outputs the reference's own class produced for the same seeded inputs."""
    stored = np.load(os.path.join(GOLDEN, "reference_cpu_outputs.npz"))[case["name"]]
    a, b, c0 = ou.golden_case_inputs(case)
    c = ou.reference_gemm(cls, case["type_in"], case["type_out"], a, b, c0, case["M"], case["N"],
                          case["K"], case["c_col_major"], case["alpha"], case["beta"])
    assert c.tobytes() == stored.tobytes()


@pytest.mark.parametrize("case", ou.GOLDEN_CPU_CASES, ids=lambda c: c["name"])
def test_matches_compiled_reference(cls, case):
    ref = ou.load_reference()
    if ref is None:
        pytest.skip("reference CPU GEMM not built on this machine")
    a, b, c0 = ou.golden_case_inputs(case)
    args = (case["type_in"], case["type_out"], a, b, c0, case["M"], case["N"], case["K"],
            case["c_col_major"], case["alpha"], case["beta"])
    assert ou.reference_gemm(cls, *args).tobytes() == ou.reference_gemm(ref, *args).tobytes()
