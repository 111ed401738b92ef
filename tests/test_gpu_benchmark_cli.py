"""The command-line benchmarks (counterparts of the reference's benchmark_gemm / _transpose /
_packing programs) run and print the reference's CSV columns."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, duration="0.05"):
    res = subprocess.run([sys.executable, "-m", "ccglib_b200.benchmark", *args, "--csv",
                          "--benchmark_duration", duration], cwd=ROOT, capture_output=True,
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


def test_gemm_cli_pad_and_power():
    """--pad rounds the sizes up to the GetDimensions tile (128, 256, 64 for float16);
    --measure_power appends the reference's two extra columns."""
    header, rows = _run("gemm", "--b", "4", "--m", "1000", "--n", "1000", "--k", "1000",
                        "--precision_in", "float16", "--pad", "--measure_power", duration="1.0")
    assert header == "#M,N,K,runtime_ms,tops,watt,tops_per_joule"
    assert rows[0][:3] == ["1024", "1024", "1024"]
    watts, tops_per_joule = float(rows[0][5]), float(rows[0][6])
    assert 10 < watts < 1500 and tops_per_joule > 0


def test_gemm_cli_multi_gpu():
    """--gpus N splits the batch over N GPUs (one host thread each) and reports the aggregate."""
    import torch

    n = min(2, torch.cuda.device_count())
    header, rows = _run("gemm", "--gpus", str(n), "--b", "5", "--m", "512", "--n", "512", "--k",
                        "1024", "--precision_in", "float16")
    assert header == "#M,N,K,runtime_ms,tops"
    assert rows[0][:3] == ["512", "512", "1024"] and float(rows[0][4]) > 0


def test_tune_cli():
    res = subprocess.run([sys.executable, "-m", "ccglib_b200.tune", "--b", "2", "--m", "512", "--n",
                          "512", "--k", "1024", "--precision_in", "float16", "--duration", "0.02"],
                         cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr
    assert "plan's choice" in res.stdout and "best fixed form" in res.stdout
    res = subprocess.run([sys.executable, "-m", "ccglib_b200.tune", "--m", "512", "--n", "512",
                          "--k", "2048", "--precision_in", "int1", "--data", "random",
                          "--duration", "0.02"], cwd=ROOT, capture_output=True, text=True,
                         timeout=300)
    assert res.returncode == 0, res.stderr
    assert "pair, 224 columns" in res.stdout
