"""Tile-shape sweep for one GEMM shape: times every kernel form the library has for it and shows
which one the plan's own model picks.  The counterpart of the reference's kernel_tuner script
(tuning/tune_gemm.py), whose search space (WMMA block and warp shapes, buffer count) does not
exist here; what can vary is the tile width (64, 128, 256 columns; 128, 192, 224 on the 1-bit
path), one CTA or a CTA pair per tile, and the operand bit pattern, which decides whether the
board's power cap binds.

    python -m ccglib_b200.tune --b 8 --m 8192 --n 8192 --k 8192 --precision_in float16
    python -m ccglib_b200.tune --b 4096 --m 256 --n 2048 --k 512 --precision_in bfloat16 --data random
    python -m ccglib_b200.tune ... --write table.json     # store the winner for the plan to use
    python -m ccglib_b200.tune ... --ncu                  # print the ncu command for one launch
    CCGLIB_B200_LIB=ccglib_b200/lib/trace/libccglib_b200.so \
        python -m ccglib_b200.tune ... --timeline         # per-tile clock stamps (instrumented build)

Every form is selected through the same environment variables a user can set for a deployment
(CCGLIB_B200_BN, CCGLIB_B200_PAIR, CCGLIB_B200_GROUP); torch only provides device memory, streams
and events.  With --write the fastest form (tile width, one CTA or a pair, column-panel width of
the tile walk) is merged into a JSON table keyed by (types, M, N, log2 bucket of the bytes per
input row, log2 bucket of the batch); a plan created while CCGLIB_B200_TUNE_TABLE names that file
takes its tile choice from it instead of the built-in model (as the reference's tuner results
select its kernel parameters, tuning/tune_gemm.py:316-363).  --ncu prints the command that
collects, for ONE launch of a small case, the DRAM byte counters the reference's tuner records
(tuning/ncu_metrics.py:4-19) plus the tensor-pipe and L2 counters that matter on this hardware.
"""
from __future__ import annotations

import argparse
import json
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
KEYS = ("CCGLIB_B200_BN", "CCGLIB_B200_PAIR", "CCGLIB_B200_INT1_MXF4", "CCGLIB_B200_GROUP",
        "CCGLIB_B200_TUNE_TABLE")
GROUPS = (2, 4, 8, 16)  # column-panel widths tried on the fastest tile form
TABLE_FORMAT = "ccglib_b200 tuning table 1"
NCU_METRICS = ("dram__bytes_read.sum,dram__bytes_write.sum,"
               "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed,"
               "lts__t_sector_hit_rate.pct,gpu__time_duration.sum")


def log2_bucket(v: int) -> int:
    b = 0
    while (1 << b) < v:
        b += 1
    return b


def table_key(tin, tout, b, m, n, k):
    """The key a plan looks a problem up by (ccglib_b200_tune_table_lookup)."""
    return {"type_in": tin, "type_out": tout, "m": m, "n": n,
            "k_bucket": log2_bucket(-(-k * BITS[tin] // 8)), "batch_bucket": log2_bucket(b)}


def merge_into_table(path, entry):
    table = {"format": TABLE_FORMAT, "entries": []}
    if os.path.exists(path):
        with open(path) as f:
            table = json.load(f)
    keys = ("type_in", "type_out", "m", "n", "k_bucket", "batch_bucket")
    table["entries"] = [e for e in table.get("entries", [])
                        if any(e.get(k) != entry[k] for k in keys)] + [entry]
    with open(path, "w") as f:
        json.dump(table, f, indent=1)


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


def _timeline(args, tin, tout, d_a, d_b, d_c, stream) -> int:
    """Mean per-tile intervals, in SM clock cycles, over the CTAs of one launch: how long the MMA
    issuer is held by a tile, how long until its accumulator is complete, how long the epilogue
    takes and how much of it delays the next tile."""
    import ctypes

    import numpy as np
    import torch

    lib = capi.lib()
    if not hasattr(lib, "ccglib_b200_debug_trace_read"):
        print("this library has no clock stamps: build it with `python -m ccglib_b200.build "
              "--trace` and select it with CCGLIB_B200_LIB", file=sys.stderr)
        return 1
    plan = capi.GemmPlan(args.b, args.m, args.n, args.k, tin, tout, variant=capi.BASIC)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(3):
        plan.run(d_a.data_ptr(), d_b.data_ptr(), d_c.data_ptr(), stream)
    e0.record()
    plan.run(d_a.data_ptr(), d_b.data_ptr(), d_c.data_ptr(), stream)
    e1.record()
    torch.cuda.synchronize()
    n = 160 * 48 * 4
    buf = (ctypes.c_longlong * n)()
    lib.ccglib_b200_debug_trace_read.argtypes = [ctypes.c_void_p, ctypes.c_size_t]
    if lib.ccglib_b200_debug_trace_read(buf, n) != 0:
        return 1
    t = np.frombuffer(buf, dtype=np.int64).reshape(160, 48, 4)
    t = t[(t[:, 40, 0] > 0)][:, 2:40]  # (leader) CTAs that ran at least 41 tiles; skip the first two
    if t.shape[0] == 0:
        print("too few tiles per CTA for a timeline (need more than 40)", file=sys.stderr)
        return 1
    ms = e0.elapsed_time(e1)
    print("%s: %.3f ms, %.1f TOps/s, %d CTAs traced" % (plan.tile, ms,
          8e-9 * args.b * args.m * args.n * args.k / ms, t.shape[0]))
    print("tile period at the MMA issuer          %8.0f clk" % (t[:, 1:, 0] - t[:, :-1, 0]).mean())
    print("tile start -> last MMA issued          %8.0f clk" % (t[:, :, 1] - t[:, :, 0]).mean())
    print("tile start -> accumulator complete     %8.0f clk" % (t[:, :, 2] - t[:, :, 0]).mean())
    print("epilogue (accumulator complete -> free) %7.0f clk" % (t[:, :, 3] - t[:, :, 2]).mean())
    print("last MMA issued -> next tile may start %8.0f clk" % (t[:, 1:, 0] - t[:, :-1, 1]).mean())
    plan.close()
    return 0


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
    ap.add_argument("--write", metavar="FILE", default=None,
                    help="merge the fastest form into this tuning table (JSON)")
    ap.add_argument("--ncu", action="store_true",
                    help="print the ncu command for a single-launch capture and exit")
    ap.add_argument("--timeline", action="store_true",
                    help="per-tile timeline of the plan's choice from the clock stamps of an "
                         "instrumented library (python -m ccglib_b200.build --trace, selected "
                         "with CCGLIB_B200_LIB)")
    ap.add_argument("--single", action="store_true",
                    help="one warm-up and one launch of the plan's choice, nothing else "
                         "(the program an ncu capture runs)")
    args = ap.parse_args(argv)
    if args.ncu:
        # one kernel, one launch, no clock locking; size the case to a few GB at most
        small_b = max(1, min(args.b, (2 << 30) // max(1, 2 * (args.m + args.n) * args.k)))
        print("ncu --clock-control none --metrics %s -k regex:cgemm -s 1 -c 1 "
              "python -m ccglib_b200.tune --single --b %d --m %d --n %d --k %d --precision_in %s "
              "--precision_out %s --data random" % (NCU_METRICS, small_b, args.m, args.n, args.k,
                                                    args.precision_in, args.precision_out))
        return 0

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
    if args.timeline:
        return _timeline(args, tin, tout, d_a, d_b, d_c, stream)
    if args.single:
        plan = capi.GemmPlan(args.b, args.m, args.n, args.k, tin, tout, variant=capi.BASIC)
        for _ in range(2):
            plan.run(d_a.data_ptr(), d_b.data_ptr(), d_c.data_ptr(), stream)
        torch.cuda.synchronize()
        print("ran twice:", plan.tile)
        return 0
    saved = {k: os.environ.get(k) for k in KEYS}
    results = []

    def time_form(label, env):
        for k in KEYS:
            os.environ.pop(k, None)
        os.environ.update(env)
        try:
            plan = capi.GemmPlan(args.b, args.m, args.n, args.k, tin, tout, variant=capi.BASIC)
        except RuntimeError as exc:
            print("%-32s not available (%s)" % (label, str(exc)[:60]))
            return None
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
        tile = plan.tile
        print("%-32s %9.4f ms %9.1f TOps/s   %s" % (
            label, ms, tops, " ".join("%s=%s" % kv for kv in env.items())))
        plan.close()
        return (label, env, ms, tops, tile)

    for label, env in (FORMS_INT1 if tin == capi.INT1 else FORMS):
        r = time_form(label, env)
        if r is not None:
            results.append(r)
    # panel widths of the tile walk on the fastest tile form
    if len(results) > 1:
        base = max(results[1:], key=lambda r: r[3])
        for g in GROUPS:
            env = dict(base[1], CCGLIB_B200_GROUP=str(g))
            r = time_form("%s, panels of %d" % (base[0], g), env)
            if r is not None:
                results.append(r)
    for k, v in saved.items():
        os.environ.pop(k, None)
        if v is not None:
            os.environ[k] = v
    if len(results) > 1:
        best = max(results[1:], key=lambda r: r[3])
        print("best fixed form: %s (%.1f TOps/s); the plan's choice reaches %.1f %% of it" % (
            best[0], best[3], 100.0 * results[0][3] / best[3]))
        if args.write:
            env, tile = best[1], best[4]
            if env.get("CCGLIB_B200_INT1_MXF4") == "0":
                print("the int8 route is an environment choice, not a table entry: nothing written")
                return 0
            entry = dict(table_key(tin, tout, args.b, args.m, args.n, args.k),
                         bn=tile["bn"], pair=tile["pair"],
                         group_n=int(env.get("CCGLIB_B200_GROUP", "0")),
                         tops=round(best[3], 1), form=best[0], data=args.data)
            merge_into_table(args.write, entry)
            print("wrote %s: %s" % (args.write, json.dumps(entry)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
