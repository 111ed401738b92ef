"""Runs the self-checking C++ program that exercises the reference-shaped C++ classes
(include/ccglib: GEMM, Transpose, Packing, Pipeline; raw CUDA handles and cu:: overloads)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tests", "cpp"))

pytestmark = pytest.mark.gpu


def test_cpp_api_program():
    import build_cpp_test as cpp_build

    exe = cpp_build.build()
    res = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    print(res.stdout)
    print(res.stderr, file=sys.stderr)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "0 failure(s)" in res.stdout
    assert res.stdout.count("PASS") >= 12
