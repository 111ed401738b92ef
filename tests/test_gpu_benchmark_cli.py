"""The command-line benchmarks (counterparts of the reference's benchmark_gemm / _transpose /
_packing programs) run and print the reference's CSV columns."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    res = subprocess.run([sys.executable, "-m", "ccglib_b200.benchmark", *args, "--csv",
                          "--benchmark_duration", "0.05"], cwd=ROOT, capture_output=True,
                         text=True, timeout=300)
    assert res.returncode == 0, res.stderr
    lines = res.stdout.strip().splitlines()
    return lines[0], [line.split(",") for line in lines[1:]]


def test_gemm_cli():
    header, rows = _run("gemm", "--b", "2", "--m", "256,512", "--n", "256,512", "--k", "256,1024",
                        "--precision_in", "float16")
    assert header == "#M,N,K,runtime_ms,tops"
    assert [r[:3] for r in rows] == [["256", "256", "256"], ["512", "512", "1024"]]
    assert all(float(r[3]) > 0 and float(r[4]) > 0 for r in rows)
    header, rows = _run("gemm", "--b", "1", "--m", "256", "--n", "256", "--k", "1024",
                        "--precision_in", "int1", "--variant", "basic")
    assert float(rows[0][4]) > 0


def test_transpose_and_packing_cli():
    header, rows = _run("transpose", "--b", "2", "--m", "1024", "--n", "1024", "--precision",
                        "float16", "--complex_axis", "interleaved")
    assert header == "#M,N,runtime_ms,gbytes_per_s" and float(rows[0][3]) > 0
    for direction in ("pack", "unpack"):
        header, rows = _run("packing", "--n", str(1 << 22), "--direction", direction)
        assert header == "#N,runtime_ms,gbytes_per_s" and float(rows[0][2]) > 0
