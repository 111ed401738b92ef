"""Command-line micro-benchmarks of the three operators, with the flags, method and output columns
of the reference's benchmark programs (benchmark/benchmark_gemm.cpp:14-50,255-323,
benchmark_transpose.cpp, benchmark_packing.cpp): one probe run to estimate the iteration count for
`--benchmark_duration` seconds, a warm-up of the same length, then CUDA-event timing of back-to-back
runs with the operands resident on the device.

    python -m ccglib_b200.benchmark gemm --b 8 --m 8192 --n 8192 --k 8192 --precision_in float16
    python -m ccglib_b200.benchmark transpose --b 8 --m 8192 --n 8192 --precision float16
    python -m ccglib_b200.benchmark packing --n 1073741824 --direction pack
    python -m ccglib_b200.benchmark gemm --gpus 8 --b 64 --m 8192 --n 8192 --k 8192 --precision_in float16

Several sizes may be given (`--m 1024,2048 --n ... --k ...`).  `--pad` rounds M, N, K up to the
tile sizes of `GetDimensions`, as the reference's flag does.  `--measure_power` adds the average
board power over the timed runs and TOps/J (the reference reads a PMT sensor,
benchmark_gemm.cpp:239-243,279-320; here the difference of NVML's total-energy counter, a read-only
query).  torch only provides device memory, streams and events; the work goes through the C ABI.
"""
from __future__ import annotations

import argparse
import sys

from . import capi

PRECISIONS = {"float32": capi.FLOAT32, "float16": capi.FLOAT16, "bfloat16": capi.BFLOAT16,
              "float8e4m3": capi.FLOAT8E4M3, "float8e5m2": capi.FLOAT8E5M2, "int1": capi.INT1,
              "int32": capi.INT32}
BITS = {capi.FLOAT32: 32, capi.FLOAT16: 16, capi.BFLOAT16: 16, capi.FLOAT8E4M3: 8,
        capi.FLOAT8E5M2: 8, capi.INT1: 1, capi.INT32: 32}


def _sizes(text: str) -> list[int]:
    return [int(x) for x in text.split(",") if x]


class _EnergyMeter:
    """Joules drawn by one GPU between start() and stop(), from NVML's millijoule counter."""

    def __init__(self, device_index: int):
        import pynvml
        import torch

        pynvml.nvmlInit()
        self._nvml = pynvml
        # torch's ordinal follows CUDA_VISIBLE_DEVICES; NVML's does not: go through the UUID
        uuid = str(torch.cuda.get_device_properties(device_index).uuid)
        self._handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())

    def start(self) -> None:
        self._mj = self._nvml.nvmlDeviceGetTotalEnergyConsumption(self._handle)

    def stop(self) -> float:
        return (self._nvml.nvmlDeviceGetTotalEnergyConsumption(self._handle) - self._mj) * 1e-3


def _time(fn, duration_s: float, warm: bool, meter: "_EnergyMeter | None" = None):
    """(ms per run, runs, watts or None): the reference's scheme with CUDA events."""
    import torch

    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    fn()
    end.record()
    torch.cuda.synchronize()
    iterations = int(1000.0 * duration_s / max(start.elapsed_time(end), 1e-3)) + 1
    if warm:
        for _ in range(iterations):
            fn()
    torch.cuda.synchronize()
    if meter is not None:
        meter.start()
    start.record()
    for _ in range(iterations):
        fn()
    end.record()
    torch.cuda.synchronize()
    joules = meter.stop() if meter is not None else None
    status = capi.device_status()
    if status:
        raise RuntimeError("device status word 0x%x" % status)
    total_ms = start.elapsed_time(end)
    # NVML refreshes the counter every few tens of milliseconds: a shorter run reads 0 J -> nan
    watts = None if joules is None else (joules / (1e-3 * total_ms) if joules > 0 else float("nan"))
    return total_ms / iterations, iterations, watts


def _ceil(a: int, b: int) -> int:
    return -(-a // b)


def _gemm_on_device(args, device: int, batch: int, barrier, out: list) -> None:
    """The GEMM timing loop of one GPU on `batch` items; appends (M, N, K, ms, watts) rows."""
    import torch

    torch.cuda.set_device(device)
    tin = PRECISIONS[args.precision_in]
    tout = PRECISIONS[args.precision_out]
    if tin == capi.INT1:
        tout = capi.INT32
    variant = capi.OPT if args.variant == "opt" else capi.BASIC
    axis = capi.INTERLEAVED if args.complex_axis == "interleaved" else capi.PLANAR
    m_blk, n_blk, k_c = capi.gemm_dims(tin, tout, variant)
    stream = int(torch.cuda.current_stream().cuda_stream)
    meter = _EnergyMeter(device) if args.measure_power else None
    dev = "cuda:%d" % device
    first = True
    for _ in range(args.nr_benchmarks):
        for M, N, K in zip(_sizes(args.m), _sizes(args.n), _sizes(args.k)):
            if args.pad:
                M, N, K = _ceil(M, m_blk) * m_blk, _ceil(N, n_blk) * n_blk, _ceil(K, k_c) * k_c
            if variant == capi.OPT:  # zero-padded tiled operands
                a_bytes = batch * 2 * _ceil(M, m_blk) * m_blk * _ceil(K, k_c) * k_c * BITS[tin] // 8
                b_bytes = batch * 2 * _ceil(N, n_blk) * n_blk * _ceil(K, k_c) * k_c * BITS[tin] // 8
            else:
                row = _ceil(K, 32) * 4 if tin == capi.INT1 else K * BITS[tin] // 8
                a_bytes, b_bytes = batch * 2 * M * row, batch * 2 * N * row
            # operand bytes: 0x3c patterns decode to small finite values in every float type
            d_a = torch.full((a_bytes,), 0x3C, dtype=torch.uint8, device=dev)
            d_b = torch.full((b_bytes,), 0x3C, dtype=torch.uint8, device=dev)
            d_c = torch.empty(batch * 2 * M * N * BITS[tout] // 8, dtype=torch.uint8, device=dev)
            plan = capi.GemmPlan(batch, M, N, K, tin, tout, variant=variant, c_complex_axis=axis)
            if barrier is not None:
                barrier.wait()  # all GPUs start the same problem together
            ms, _, watts = _time(
                lambda: plan.run(d_a.data_ptr(), d_b.data_ptr(), d_c.data_ptr(), stream),
                args.benchmark_duration, first, meter)
            first = False
            out.append((M, N, K, ms, watts))
            plan.close()
            del d_a, d_b, d_c


def bench_gemm(args) -> None:
    """One GPU (`--device`), or `--gpus N`: the batch is split over GPUs 0..N-1 in contiguous
    shares (the partition `bench.py` uses), one host thread per GPU, no data-path collective;
    the reported time is the slowest GPU's and the rate is the whole batch over that time."""
    import threading

    from .sharding import batch_shares

    power = args.measure_power
    capi.lib()  # load the library before any thread needs it
    if args.csv:
        print("#M,N,K,runtime_ms,tops" + (",watt,tops_per_joule" if power else ""))
    if args.gpus <= 1:
        rows: list = []
        _gemm_on_device(args, args.device, args.b, None, rows)
        per_gpu = [rows]
    else:
        shares = [n for n in batch_shares(args.b, args.gpus) if n > 0]
        barrier = threading.Barrier(len(shares))
        per_gpu = [[] for _ in shares]
        errors: list = []

        def work(g):
            try:
                _gemm_on_device(args, g, shares[g], barrier, per_gpu[g])
            except BaseException as exc:  # surface the failure instead of a hung barrier
                errors.append(exc)
                barrier.abort()

        threads = [threading.Thread(target=work, args=(g,)) for g in range(len(shares))]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        if errors:
            raise errors[0]
    for i, (M, N, K, _, _) in enumerate(per_gpu[0]):
        ms = max(rows[i][3] for rows in per_gpu)
        tops = 8e-9 * args.b * M * N * K / ms
        watts = sum(rows[i][4] for rows in per_gpu) if power else None
        if args.csv:
            print("%d,%d,%d,%g,%g" % (M, N, K, ms, tops) +
                  (",%g,%g" % (watts, tops / watts) if power else ""))
        else:
            print("%20s %7.4g ms, %7.4g TOps/s" % ("%dx%dx%d" % (M, N, K), ms, tops) +
                  (", %7.4g W, %7.4g TOps/J" % (watts, tops / watts) if power else ""))


def bench_transpose(args) -> None:
    import torch

    t = PRECISIONS[args.precision]
    bits = BITS[t]
    tout = capi.INT32 if t == capi.INT1 else capi.FLOAT32
    variant = capi.OPT if args.variant == "opt" else capi.BASIC
    axis = capi.INTERLEAVED if args.complex_axis == "interleaved" else capi.PLANAR
    m_blk, _, k_c = capi.gemm_dims(t, tout, variant)
    stream = int(torch.cuda.current_stream().cuda_stream)
    meter = _EnergyMeter(args.device) if args.measure_power else None
    if args.csv:
        print("#M,N,runtime_ms,gbytes_per_s" + (",watt" if meter else ""))
    first = True
    for _ in range(args.nr_benchmarks):
        for M, N in zip(_sizes(args.m), _sizes(args.n)):
            in_bytes = args.b * 2 * M * N * bits // 8
            out_bytes = args.b * 2 * _ceil(M, m_blk) * m_blk * _ceil(N, k_c) * k_c * bits // 8
            d_in = torch.full((in_bytes,), 0x3C, dtype=torch.uint8, device="cuda")
            d_out = torch.empty(out_bytes, dtype=torch.uint8, device="cuda")
            ms, _, watts = _time(lambda: capi.transpose(args.b, M, N, m_blk, k_c, bits, axis,
                                                        d_in.data_ptr(), d_out.data_ptr(), stream),
                                 args.benchmark_duration, first, meter)
            first = False
            gbs = 2e-6 * in_bytes / ms  # bytes read + bytes written, padding not counted
            if args.csv:
                print("%d,%d,%g,%g" % (M, N, ms, gbs) + (",%g" % watts if meter else ""))
            else:
                print("%20s %7.4g ms, %7.4g GByte/s" % ("%dx%d" % (M, N), ms, gbs) +
                      (", %7.4g W" % watts if meter else ""))
            del d_in, d_out


def bench_packing(args) -> None:
    import torch

    direction = capi.FORWARD if args.direction == "pack" else capi.BACKWARD
    stream = int(torch.cuda.current_stream().cuda_stream)
    meter = _EnergyMeter(args.device) if args.measure_power else None
    if args.csv:
        print("#N,runtime_ms,gbytes_per_s" + (",watt" if meter else ""))
    first = True
    for _ in range(args.nr_benchmarks):
        for N in _sizes(args.n):
            byte_side = torch.ones(N, dtype=torch.uint8, device="cuda")
            word_side = torch.zeros(_ceil(N, 32) * 4, dtype=torch.uint8, device="cuda")
            src, dst = (byte_side, word_side) if direction == capi.FORWARD else (word_side,
                                                                               byte_side)
            ms, _, watts = _time(lambda: capi.pack(N, direction, capi.PLANAR, src.data_ptr(),
                                                   dst.data_ptr(), stream),
                                 args.benchmark_duration, first, meter)
            first = False
            gbs = 1e-6 * (N + N / 8) / ms
            if args.csv:
                print("%d,%g,%g" % (N, ms, gbs) + (",%g" % watts if meter else ""))
            else:
                print("%20d %7.4g ms, %7.4g GByte/s" % (N, ms, gbs) +
                      (", %7.4g W" % watts if meter else ""))
            del byte_side, word_side


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m ccglib_b200.benchmark")
    sub = ap.add_subparsers(dest="what", required=True)

    def common(p):
        p.add_argument("--nr_benchmarks", type=int, default=1)
        p.add_argument("--benchmark_duration", type=float, default=4.0)
        p.add_argument("--csv", action="store_true")
        p.add_argument("--device", type=int, default=0)
        p.add_argument("--measure_power", action="store_true")

    g = sub.add_parser("gemm")
    g.add_argument("--b", type=int, default=1)
    g.add_argument("--m", required=True)
    g.add_argument("--n", required=True)
    g.add_argument("--k", required=True)
    g.add_argument("--pad", action="store_true")
    g.add_argument("--gpus", type=int, default=1,
                   help="split the batch over this many GPUs (0..N-1), one host thread each")
    g.add_argument("--precision_in", default="float32", choices=sorted(PRECISIONS))
    g.add_argument("--precision_out", default="float32", choices=sorted(PRECISIONS))
    g.add_argument("--variant", default="opt", choices=["basic", "opt"])
    g.add_argument("--complex_axis", default="planar", choices=["planar", "interleaved"])
    common(g)
    t = sub.add_parser("transpose")
    t.add_argument("--b", type=int, default=1)
    t.add_argument("--m", required=True)
    t.add_argument("--n", required=True)
    t.add_argument("--precision", required=True, choices=sorted(PRECISIONS))
    t.add_argument("--variant", default="opt", choices=["basic", "opt"])
    t.add_argument("--complex_axis", default="planar", choices=["planar", "interleaved"])
    common(t)
    p = sub.add_parser("packing")
    p.add_argument("--n", required=True)
    p.add_argument("--direction", default="pack", choices=["pack", "unpack"])
    common(p)
    args = ap.parse_args(argv)

    import torch

    if not torch.cuda.is_available():
        print("a CUDA device is required", file=sys.stderr)
        return 1
    torch.cuda.set_device(args.device)
    {"gemm": bench_gemm, "transpose": bench_transpose, "packing": bench_packing}[args.what](args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
