"""Pins the CPU oracle (oracle/oracle.c) against the reference's own known-answer vectors
(test/gemm/reference.cpp, read into tests/golden/reference_test_vectors.json), against stored
outputs of the reference's own CPU GEMM on seeded inputs, and -- where the reference CPU GEMM
could be compiled here -- against that binary directly."""
import json
import os

import numpy as np
import pytest

import oracle_util as ou

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
VECTORS = json.load(open(os.path.join(GOLDEN, "reference_test_vectors.json")))
NAME_TO_TYPE = {"float16": ou.F16, "bfloat16": ou.BF16, "float32": ou.F32}


@pytest.mark.parametrize("type_name", VECTORS["float"]["input_types"])
@pytest.mark.parametrize("col", [False, True])
def test_float_known_answer(type_name, col):
    v = VECTORS["float"]
    t = NAME_TO_TYPE[type_name]
    M, N, K = v["M"], v["N"], v["K"]
    a = ou.quantize(np.array(v["a"], np.float32).reshape(2, M, K), t)
    b = ou.quantize(np.array(v["b"], np.float32).reshape(2, N, K), t)
    c = ou.port_gemm(t, ou.F32, a, b, None, M, N, K, c_col_major=col)
    want = np.array(v["c_col_major" if col else "c_row_major"], np.float32)
    assert np.array_equal(c.ravel(), want)


@pytest.mark.parametrize("col", [False, True])
def test_binary_known_answer(col):
    v = VECTORS["binary"]
    M, N, K = v["M"], v["N"], v["K"]
    a = np.array(v["a"], np.uint32).reshape(2, M, K // 32)
    b = np.array(v["b"], np.uint32).reshape(2, N, K // 32)
    c = ou.port_gemm(ou.INT1, ou.INT32, a, b, None, M, N, K, c_col_major=col)
    assert c.ravel().tolist() == v["c_col_major" if col else "c_row_major"]


def test_alpha_beta_float16_known_answer():
    v = VECTORS["alpha_beta_float16"]
    M, N, K = v["M"], v["N"], v["K"]
    a = ou.quantize(np.array(v["a"], np.float32).reshape(2, M, K), ou.F16)
    b = ou.quantize(np.array(v["b"], np.float32).reshape(2, N, K), ou.F16)
    c0 = np.array(v["c_in"], np.float32).reshape(2, M, N)
    c = ou.port_gemm(ou.F16, ou.F32, a, b, c0, M, N, K, alpha=tuple(v["alpha"]),
                     beta=tuple(v["beta"]))
    assert np.array_equal(c.ravel(), np.array(v["c_ref"], np.float32))


def test_alpha_beta_int1_known_answer():
    v = VECTORS["alpha_beta_int1"]
    M, N, K = v["M"], v["N"], v["K"]
    a = np.array(v["a"], np.uint32).reshape(2, M, K // 32)
    b = np.array(v["b"], np.uint32).reshape(2, N, K // 32)
    c0 = np.array(v["c_in"], np.int32).reshape(2, M, N)
    c = ou.port_gemm(ou.INT1, ou.INT32, a, b, c0, M, N, K, alpha=tuple(v["alpha"]),
                     beta=tuple(v["beta"]))
    assert c.ravel().tolist() == v["c_ref"]


@pytest.mark.parametrize("case", ou.GOLDEN_CPU_CASES, ids=lambda c: c["name"])
def test_port_matches_stored_reference_outputs(case):
    stored = np.load(os.path.join(GOLDEN, "reference_cpu_outputs.npz"))[case["name"]]
    a, b, c0 = ou.golden_case_inputs(case)
    c = ou.port_gemm(case["type_in"], case["type_out"], a, b, c0, case["M"], case["N"], case["K"],
                     case["c_col_major"], case["alpha"], case["beta"])
    assert c.tobytes() == stored.tobytes()


@pytest.mark.parametrize("case", ou.GOLDEN_CPU_CASES, ids=lambda c: c["name"])
def test_port_matches_compiled_reference(case):
    ref = ou.load_reference()
    if ref is None:
        pytest.skip("reference CPU GEMM not built on this machine")
    a, b, c0 = ou.golden_case_inputs(case)
    args = (case["type_in"], case["type_out"], a, b, c0, case["M"], case["N"], case["K"],
            case["c_col_major"], case["alpha"], case["beta"])
    assert ou.port_gemm(*args).tobytes() == ou.reference_gemm(ref, *args).tobytes()


def test_widen_matches_numpy_and_torch():
    import torch

    h = np.arange(0, 1 << 16, dtype=np.uint16)
    got = ou.widen(h.view(np.float16), ou.F16)
    want = h.view(np.float16).astype(np.float32)
    assert np.array_equal(got.view(np.uint32)[~np.isnan(want)], want.view(np.uint32)[~np.isnan(want)])
    b8 = np.arange(256, dtype=np.uint8)
    for vt, dt in ((ou.E4M3, torch.float8_e4m3fn), (ou.E5M2, torch.float8_e5m2)):
        want = torch.from_numpy(b8.copy()).view(dt).to(torch.float32).numpy()
        got = ou.widen(b8, vt)
        ok = ~np.isnan(want)
        assert np.array_equal(got[ok], want[ok]) and np.all(np.isnan(got[~ok]))
    want = torch.from_numpy(h.view(np.int16).copy()).view(torch.bfloat16).to(torch.float32).numpy()
    got = ou.widen(h, ou.BF16)
    ok = ~np.isnan(want)
    assert np.array_equal(got[ok], want[ok])


def test_narrow_round_to_nearest_even():
    import torch

    rng = np.random.default_rng(5)
    x = np.concatenate([rng.standard_normal(20000).astype(np.float32) * s
                        for s in (1e-8, 1e-5, 1e-3, 1.0, 100.0, 7e4)])
    x = np.concatenate([x, np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 2.0**-24, 2.0**-25,
                                     2.0**-25 * 1.0001, 5.9604645e-08 * 1.5], np.float32)])
    assert np.array_equal(ou.narrow(x, ou.F16).view(np.uint16), x.astype(np.float16).view(np.uint16))
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(ou.narrow(x, ou.BF16), want)


def test_pack_unpack_roundtrip_and_bit_order():
    rng = np.random.default_rng(7)
    n = 2048 + 13
    x = rng.integers(0, 2, n).astype(np.uint8)
    w = ou.port_pack(x)
    for i in (0, 1, 31, 32, 100, n - 1):
        assert (w[i // 32] >> (i % 32)) & 1 == x[i]
    assert np.array_equal(ou.port_unpack(w, n), x)
    # interleaved input: [n/2][2] -> planar [2][n/2]
    n = 2048
    x = rng.integers(0, 2, n).astype(np.uint8)
    planar = np.ascontiguousarray(x.reshape(n // 2, 2).T).ravel()
    assert np.array_equal(ou.port_pack(x, interleaved=True), ou.port_pack(planar))


@pytest.mark.parametrize("bits,interleaved", [(16, False), (16, True), (8, False), (32, True),
                                              (1, False)])
def test_transpose_index_formula(bits, interleaved):
    # the layout the reference's transpose test checks (test/transpose/transpose.cpp:113-146)
    rng = np.random.default_rng(bits)
    B, M, N, Mc, Nc = 2, 70, 96, 32, 64
    dt = {1: np.uint32, 8: np.uint8, 16: np.uint16, 32: np.uint32}[bits]
    n_el, nc_el = (N // 32, Nc // 32) if bits == 1 else (N, Nc)
    shape = (B, M, n_el, 2) if interleaved else (B, 2, M, n_el)
    x = rng.integers(1, 255, size=shape).astype(dt)
    out = ou.port_transpose(x.ravel(), B, M, N, Mc, Nc, bits, interleaved)
    mt, nt = -(-M // Mc), -(-n_el // nc_el)
    out = out.reshape(B, mt, nt, 2, Mc, nc_el)
    planar = np.moveaxis(x, 3, 1) if interleaved else x
    want = np.zeros((B, mt, nt, 2, Mc, nc_el), dt)
    for m in range(M):
        for n in range(n_el):
            want[:, m // Mc, n // nc_el, :, m % Mc, n % nc_el] = planar[:, :, m, n]
    assert np.array_equal(out, want)
