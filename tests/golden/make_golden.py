"""Generate the golden fixtures that pin the CPU oracle.

Run where the reference checkout is available (its location is taken from the environment
variable ``CCGLIB_REFERENCE_ROOT``, see oracle/build.py):

    python tests/golden/make_golden.py

Writes, next to this file:

* ``reference_test_vectors.json`` -- the known-answer vectors of the reference's
  own oracle tests, read as text from ``test/gemm/reference.cpp`` (3x2x2 complex
  float GEMM row/col-major :27-45, 2x2x32 binary GEMM :73-80, fp16 alpha/beta
  :98-113, int1 alpha/beta :121-137).  Nothing is typed in by hand.
* ``reference_cpu_outputs.npz`` -- outputs of the reference's own CPU GEMM
  (``src/reference/GEMM.cpp`` compiled unmodified by ``oracle/build.py``) on small
  seeded inputs; the inputs are regenerated from the seed by
  ``tests/oracle_util.py`` so only the outputs are stored.
"""
from __future__ import annotations

import json
import os
import re
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def _numbers(text: str) -> list[float]:
    text = re.sub(r"static_cast<\w+>\(([^)]*)\)", r"\1", text)
    return [float(x) for x in re.findall(r"-?\d+(?:\.\d+)?", text)]


def _array(src: str, name: str, start: int = 0) -> tuple[list[float], int]:
    """Return the brace-initialiser of the first variable `name` after `start`."""
    m = re.compile(r"\b" + re.escape(name) + r"\b[^;{]*\{").search(src, start)
    if m is None:
        raise RuntimeError(f"{name} not found")
    end = src.index("}", m.end())
    return _numbers(src[m.end():end]), end


def _scalar(src: str, name: str, start: int = 0) -> tuple[list[float], int]:
    m = re.compile(r"\b" + re.escape(name) + r"\s*=\s*([^;]*);").search(src, start)
    if m is None:
        raise RuntimeError(f"{name} not found")
    return _numbers(m.group(1)), m.end()


def parse_reference_tests(path: str) -> dict:
    src = open(path).read()
    out = {"source": "test/gemm/reference.cpp"}

    # float test (templated over half, bf16, float)
    pos = src.index("runTestReference")
    dims = {}
    for d in "MNK":
        dims[d], _ = _scalar(src, f"size_t {d}", pos)
    a, p = _array(src, "a", pos)
    b, p = _array(src, "b", p)
    c_row, p = _array(src, "c_ref_row_major", p)
    c_col, p = _array(src, "c_ref_col_major", p)
    out["float"] = {"M": int(dims["M"][0]), "N": int(dims["N"][0]), "K": int(dims["K"][0]),
                    "a": a, "b": b, "c_row_major": c_row, "c_col_major": c_col,
                    "input_types": ["float16", "bfloat16", "float32"]}

    # binary test
    pos = src.index('TEST_CASE("Reference complex binary")')
    dims = {}
    for d in "MNK":
        dims[d], _ = _scalar(src, f"size_t {d}", pos)
    a, p = _array(src, "a = new unsigned", pos)
    b, p = _array(src, "b = new unsigned", p)
    c_row, p = _array(src, "c_ref_row_major", p)
    c_col, p = _array(src, "c_ref_col_major", p)
    out["binary"] = {"M": int(dims["M"][0]), "N": int(dims["N"][0]), "K": int(dims["K"][0]),
                     "a": [int(x) for x in a], "b": [int(x) for x in b],
                     "c_row_major": [int(x) for x in c_row], "c_col_major": [int(x) for x in c_col]}

    # alpha/beta float16
    pos = src.index('SECTION("float16")')
    dims = {}
    for d in "MNK":
        dims[d], _ = _scalar(src, f"size_t {d}", pos)
    alpha, _ = _scalar(src, "alpha", pos)
    beta, _ = _scalar(src, "beta", pos)
    a, p = _array(src, "half a", pos)
    b, p = _array(src, "half b", p)
    c_in, p = _array(src, "c_test", p)
    c_ref, p = _array(src, "c_ref", p)
    out["alpha_beta_float16"] = {"M": int(dims["M"][0]), "N": int(dims["N"][0]),
                                 "K": int(dims["K"][0]), "alpha": alpha, "beta": beta,
                                 "a": a, "b": b, "c_in": c_in, "c_ref": c_ref}

    # alpha/beta int1
    pos = src.index('SECTION("int1")')
    dims = {}
    for d in "MNK":
        dims[d], _ = _scalar(src, f"size_t {d}", pos)
    alpha, _ = _scalar(src, "alpha", pos)
    beta, _ = _scalar(src, "beta", pos)
    a, p = _array(src, "a = new unsigned", pos)
    b, p = _array(src, "b = new unsigned", p)
    c_in, p = _array(src, "c_test", p)
    c_ref, p = _array(src, "c_ref", p)
    out["alpha_beta_int1"] = {"M": int(dims["M"][0]), "N": int(dims["N"][0]),
                              "K": int(dims["K"][0]), "alpha": alpha, "beta": beta,
                              "a": [int(x) for x in a], "b": [int(x) for x in b],
                              "c_in": [int(x) for x in c_in], "c_ref": [int(x) for x in c_ref]}
    return out


def reference_cpu_outputs() -> dict:
    import oracle_util as ou

    ref = ou.load_reference()
    if ref is None:
        raise RuntimeError("reference CPU GEMM library not built (python oracle/build.py)")
    out = {}
    for case in ou.GOLDEN_CPU_CASES:
        a, b, c0 = ou.golden_case_inputs(case)
        c = ou.reference_gemm(ref, case["type_in"], case["type_out"], a, b, c0, case["M"],
                              case["N"], case["K"], case["c_col_major"], case["alpha"],
                              case["beta"])
        out[case["name"]] = c.view(np.uint8) if c.dtype.itemsize == 1 else c
    return out


def main() -> None:
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import build as oracle_build

    ref_root = oracle_build.reference_root()
    vectors = parse_reference_tests(os.path.join(ref_root, "test", "gemm", "reference.cpp"))
    with open(os.path.join(HERE, "reference_test_vectors.json"), "w") as f:
        json.dump(vectors, f, indent=1)
    oracle_build.build_all()
    np.savez_compressed(os.path.join(HERE, "reference_cpu_outputs.npz"), **reference_cpu_outputs())
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
