"""Tile-shape sweep for one GEMM shape: times every kernel form the library has for it and shows
which one the plan's own model picks.  The counterpart of the reference's kernel_tuner script
(tuning/tune_gemm.py), whose search space (WMMA block and warp shapes, buffer count) does not
exist here; what can vary is the tile width (64, 128, 256 columns; 128, 192, 224 on the 1-bit
path), one CTA or a CTA pair per tile, and the operand bit pattern, which decides whether the
board's power cap binds.

    python -m ccglib_b200.tune --b 8 --m 8192 --n 8192 --k 8192 --precision_in float16
    python -m ccglib_b200.tune --b 4096 --m 256 --n 2048 --k 512 --precision_in bfloat16 --data random

Every form is selected through the same environment variables a user can set for a deployment
(CCGLIB_B200_BN, CCGLIB_B200_PAIR); torch only provides device memory, streams and events.
"""
from __future__ import annotations

import argparse
import os
import sys

from . import capi
from .benchmark import BITS, PRECISIONS

FORMS = [  # (label, environment overrides)
    ("plan's choice", {}),
    ("1 CTA, 64 columns", {"CCGLIB_B200_BN": "64", "CCGLIB_B200_PAIR": "0"}),
    ("1 CTA, 128 columns", {"CCGLIB_B200_BN": "128", "CCGLIB_B200_PAIR": "0"}),
    ("1 CTA, 256 columns", {"CCGLIB_B200_BN": "256", "CCGLIB_B200_PAIR": "0"}),
    ("pair, 128 columns", {"CCGLIB_B200_BN": "128", "CCGLIB_B200_PAIR": "1"}),
    ("pair, 256 columns", {"CCGLIB_B200_BN": "256", "CCGLIB_B200_PAIR": "1"}),
]
FORMS_INT1 = [
    ("plan's choice", {}),
    ("pair, 128 columns", {"CCGLIB_B200_BN": "128"}),
    ("pair, 192 columns", {"CCGLIB_B200_BN": "192"}),
    ("pair, 224 columns", {"CCGLIB_B200_BN": "224"}),
    ("1 CTA, 192 columns", {"CCGLIB_B200_BN": "192", "CCGLIB_B200_PAIR": "0"}),
    ("int8 route, 1 CTA, 256 columns", {"CCGLIB_B200_INT1_MXF4": "0"}),
]
KEYS = ("CCGLIB_B200_BN", "CCGLIB_B200_PAIR", "CCGLIB_B200_INT1_MXF4")


def _operands(args, tin, row_bytes):
    import torch

    n_a, n_b = args.b * 2 * args.m * row_bytes, args.b * 2 * args.n * row_bytes
    if args.data == "constant":  # the fill of the reference's benchmark programs
        return (torch.full((n_a,), 0x3C, dtype=torch.uint8, device="cuda"),
                torch.full((n_b,), 0x3C, dtype=torch.uint8, device="cuda"))
    g = torch.Generator(device="cuda")
    g.manual_seed(7)
    out = []
    for n in (n_a, n_b):
        if tin in (capi.FLOAT16, capi.BFLOAT16, capi.FLOAT32):
            dt = {capi.FLOAT16: torch.float16, capi.BFLOAT16: torch.bfloat16,
                  capi.FLOAT32: torch.float32}[tin]
            x = (torch.randn(n // (BITS[tin] // 8), device="cuda", generator=g) /
                 max(1.0, args.k) ** 0.5).to(dt)
            out.append(x.view(torch.uint8))
        else:  # fp8 (top exponent bit cleared: finite values) and packed 1-bit words
            x = torch.randint(0, 256, (n,), device="cuda", generator=g, dtype=torch.uint8)
            out.append(x if tin == capi.INT1 else x & 0xBF)
    return out[0], out[1]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m ccglib_b200.tune")
    ap.add_argument("--b", type=int, default=1)
    ap.add_argument("--m", type=int, required=True)
    ap.add_argument("--n", type=int, required=True)
    ap.add_argument("--k", type=int, required=True)
    ap.add_argument("--precision_in", default="float16", choices=sorted(PRECISIONS))
    ap.add_argument("--precision_out", default="float32", choices=sorted(PRECISIONS))
    ap.add_argument("--data", default="constant", choices=["constant", "random"])
    ap.add_argument("--duration", type=float, default=1.0, help="seconds per form")
    ap.add_argument("--device", type=int, default=0)
    args = ap.parse_args(argv)

    import torch

    if not torch.cuda.is_available():
        print("a CUDA device is required", file=sys.stderr)
        return 1
    torch.cuda.set_device(args.device)
    tin = PRECISIONS[args.precision_in]
    tout = capi.INT32 if tin == capi.INT1 else PRECISIONS[args.precision_out]
    row_bytes = -(-args.k // 32) * 4 if tin == capi.INT1 else args.k * BITS[tin] // 8
    d_a, d_b = _operands(args, tin, row_bytes)
    d_c = torch.empty(args.b * 2 * args.m * args.n * BITS[tout] // 8, dtype=torch.uint8,
                      device="cuda")
    stream = int(torch.cuda.current_stream().cuda_stream)
    saved = {k: os.environ.get(k) for k in KEYS}
    results = []
    for label, env in (FORMS_INT1 if tin == capi.INT1 else FORMS):
        for k in KEYS:
            os.environ.pop(k, None)
        os.environ.update(env)
        try:
            plan = capi.GemmPlan(args.b, args.m, args.n, args.k, tin, tout, variant=capi.BASIC)
        except RuntimeError as exc:
            print("%-32s not available (%s)" % (label, str(exc)[:60]))
            continue
        run = lambda: plan.run(d_a.data_ptr(), d_b.data_ptr(), d_c.data_ptr(), stream)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(3):
            run()
        e0.record()
        run()
        e1.record()
        torch.cuda.synchronize()
        reps = max(3, int(1000.0 * args.duration / max(e0.elapsed_time(e1), 1e-3)))
        e0.record()
        for _ in range(reps):
            run()
        e1.record()
        torch.cuda.synchronize()
        if capi.device_status():
            raise RuntimeError("device status word set")
        ms = e0.elapsed_time(e1) / reps
        tops = 8e-9 * args.b * args.m * args.n * args.k / ms
        results.append((label, env, ms, tops))
        print("%-32s %9.4f ms %9.1f TOps/s   %s" % (
            label, ms, tops, " ".join("%s=%s" % kv for kv in env.items())))
        plan.close()
    for k, v in saved.items():
        os.environ.pop(k, None)
        if v is not None:
            os.environ[k] = v
    if len(results) > 1:
        best = max(results[1:], key=lambda r: r[3])
        print("best fixed form: %s (%.1f TOps/s); the plan's choice reaches %.1f %% of it" % (
            best[0], best[3], 100.0 * results[0][3] / best[3]))
    return 0


if __name__ == "__main__":
    sys.exit(main())
