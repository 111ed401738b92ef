"""Benchmark of the complex-GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one pass of the hot path over the whole (per-rank share of the) workload through
the library's Pipeline object (ccglib_b200_pipeline_run): for the headline workload, the optimized
fp16 -> fp32 complex GEMM on interleaved input, batch 64, M = N = K = 8192, that is Transpose(A),
Transpose(B), GEMM on one stream.  Metric: complex TOPS = 8*M*N*K*batch / time (the reference's
benchmark/benchmark_gemm.cpp:79-82).

* `value`    inputs resident in HBM, CUDA-event time of K steps, max over ranks.
* `e2e`      the same pass with HOST buffers through ccglib_b200_pipeline_run_host: the whole A, B
             and C live in pinned host memory, the library copies batch slices in, runs them and
             copies C back, double-buffered; wall clock around K blocking calls.
* `roofline` the GEMM stage alone: 8*M*N*K*batch flops per launch / its CUDA-event duration,
             against the measured tensor peak in MEASURED_PEAKS.json (and the HBM roof).
* `per_workload` the other configurations of the baseline, each device-timed for about two
             seconds with its own roofline, parity and clock record, and `reference_gpu`: the
             reference's own legacy kernel (compiled unmodified for sm_100a) timed on the same
             device and inputs for one batch slice, as a reported baseline and second checker.
* `cpu_baseline` / `--impl reference`: the reference's own CPU GEMM (oracle/_ref, else the C
             restatement in oracle/) on a bounded sample with all host threads.

With N > 1 (torchrun) the batch is split across ranks; there is no collective on the data path.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

import numpy as np  # noqa: E402

NOMINAL_TFLOPS = {"f16": 2250.0, "bf16": 2250.0, "tf32": 1125.0, "e4m3": 4500.0, "e5m2": 4500.0,
                  "int1": 9000.0}  # dense; int1 runs on the block-scaled 4-bit (e2m1) path

# name: (dtype, type_in, type_out, batch, M, N, K, variant, input layout)
WORKLOADS = {
    "c1_f16_basic_1024": ("f16", "F16", "F32", 1, 1024, 1024, 1024, "basic", "planar"),
    "c2_f16_opt_8192_b64": ("f16", "F16", "F32", 64, 8192, 8192, 8192, "opt", "interleaved"),
    # 1-bit: one byte per sample, as the reference's Pipeline takes it; the library turns the
    # bytes into tensor-core operands itself (no Packing or Transpose pass)
    "c3_int1_4096_k65536_b32": ("int1", "INT1", "INT32", 32, 4096, 4096, 65536, "opt", "bytes"),
    "c4_e4m3_4096_k16384_b32": ("e4m3", "E4M3", "F32", 32, 4096, 4096, 16384, "opt", "planar"),
    "c4_e5m2_4096_k16384_b32": ("e5m2", "E5M2", "F32", 32, 4096, 4096, 16384, "opt", "planar"),
    "c5_bf16_256x2048x512_b4096": ("bf16", "BF16", "F32", 4096, 256, 2048, 512, "basic", "planar"),
    "c5_tf32_256x2048x512_b4096": ("tf32", "F32", "F32", 4096, 256, 2048, 512, "basic", "planar"),
}
DEFAULT_WORKLOAD = "c2_f16_opt_8192_b64"

# the reference's own GPU kernel compiled for one batch slice of each workload
# (oracle/build_reference_gpu.py: CASES)
REFERENCE_GPU_CASE = {
    "c1_f16_basic_1024": "c1_f16_basic", "c2_f16_opt_8192_b64": "c2_f16_opt_b2",
    "c3_int1_4096_k65536_b32": "c3_int1_opt_b1", "c4_e4m3_4096_k16384_b32": "c4_e4m3_opt_b2",
    "c4_e5m2_4096_k16384_b32": "c4_e5m2_opt_b2",
    "c5_bf16_256x2048x512_b4096": "c5_bf16_basic_b64",
    "c5_tf32_256x2048x512_b4096": "c5_tf32_basic_b64",
}

# value-type codes of the C ABI (= the reference's ValueType ordinals) and their widths in bits
TYPE_CODE = {"INT1": 0, "INT32": 1, "BF16": 2, "E4M3": 3, "E5M2": 4, "F16": 5, "F32": 6}
TYPE_BITS = {0: 1, 1: 32, 2: 16, 3: 8, 4: 8, 5: 16, 6: 32}

# DRAM bytes (read + write) of one GEMM-kernel launch per batch item, from single-launch ncu
# captures of small cases (dram__bytes_read.sum + dram__bytes_write.sum; batch items are walked
# one after another, so the traffic grows in proportion to the batch).  Workloads without a
# capture report null.
NCU_DRAM_BYTES_PER_ITEM = {
    "c2_f16_opt_8192_b64": 3.39e9,          # 6.79 GB for a 2-item launch
    "c3_int1_4096_k65536_b32": 1.625e9,     # GEMM kernel alone: 3.25 GB for a 2-item launch
    "c4_e4m3_4096_k16384_b32": 0.8525e9,    # 3.41 GB for a 4-item launch
    "c5_bf16_256x2048x512_b4096": 9.18e6,   # 4.70 GB for a 512-item launch (= algorithmic)
}
C1_ROTATE = 16  # config 1 (16 MiB per problem) rotates over 16 operand sets: 256 MiB > L2


def measured_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        d["source"] = "measured"
        return d
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


# --------------------------------------------------------------------------- clocks sampling

class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines: list[str] = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + self.QUERY,
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(smax)),
                "power_w_max": float(max(power)), "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- CPU baseline

def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_baseline(type_in_name: str, type_out_name: str, K: int, target_s: float = 12.0) -> dict:
    """Times the reference's own CPU GEMM (or the C restatement) on a bounded sample: one batch
    item of the workload's dtype and K with M = N chosen so the run takes about target_s.  The
    OpenMP thread count is set explicitly (launchers such as torchrun export OMP_NUM_THREADS=1)
    and the count the runtime reports back is what `cores` states."""
    import oracle_util as ou

    type_in = getattr(ou, type_in_name)
    type_out = getattr(ou, type_out_name)
    want = host_threads()
    os.environ["OMP_NUM_THREADS"] = str(want)  # before the OpenMP runtime of the oracle loads
    ref = ou.load_reference()
    kind = "reference" if ref is not None else "port"
    if ref is not None:
        ref.ref_omp_set_threads(want)
        cores = int(ref.ref_omp_max_threads())
    else:
        port = ou.load_port()
        port.oracle_omp_set_threads(want)
        cores = int(port.oracle_omp_max_threads())
    rng = np.random.default_rng(7)

    def run(M, N, Kk):
        if type_in == ou.INT1:
            a = ou.random_storage(rng, (2, M, Kk // 32), ou.INT1)
            b = ou.random_storage(rng, (2, N, Kk // 32), ou.INT1)
        else:
            a = ou.random_storage(rng, (2, M, Kk), type_in, "normal", 1.0 / math.sqrt(Kk))
            b = ou.random_storage(rng, (2, N, Kk), type_in, "normal", 1.0 / math.sqrt(Kk))
        t0 = time.perf_counter()
        if ref is not None:
            ou.reference_gemm(ref, type_in, type_out, a, b, None, M, N, Kk)
        else:
            ou.port_gemm(type_in, type_out, a, b, None, M, N, Kk)
        return time.perf_counter() - t0

    probe_k = min(K, 2048)
    t = run(128, 128, probe_k)
    rate = 8.0 * 128 * 128 * probe_k / max(t, 1e-6)  # ops/s
    mn = int(math.sqrt(target_s * rate / (8.0 * K)))
    mn = max(128, min(4096, (mn // 128) * 128))
    t = run(mn, mn, K)
    ops = 8.0 * mn * mn * K
    return {"value": ops / t / 1e12, "unit": "TOPS", "cores": cores, "kind": kind,
            "sample": "1 batch item, M=N=%d, K=%d, %s->%s, %.1f s, %d OpenMP threads" % (
                mn, K, type_in_name.lower(), type_out_name.lower(), t, cores),
            "seconds": t}


# --------------------------------------------------------------------------- device workload

def _torch_dtype(torch, dtype):
    return {"f16": torch.float16, "bf16": torch.bfloat16, "tf32": torch.float32,
            "e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}[dtype]


class Workload:
    """Device-resident operands of one workload and its Pipeline (the library object whose
    run() is one step)."""

    def __init__(self, name: str, batch: int, device):
        import torch

        from ccglib_b200 import capi

        self.torch, self.capi = torch, capi
        dtype, tin, tout, _, M, N, K, variant, layout = WORKLOADS[name]
        self.name, self.dtype, self.B, self.M, self.N, self.K = name, dtype, batch, M, N, K
        self.type_in, self.type_out = TYPE_CODE[tin], TYPE_CODE[tout]
        self.variant = capi.OPT if variant == "opt" else capi.BASIC
        self.layout = layout
        self.device = device
        self.bits = TYPE_BITS[self.type_in]
        # config 1 is one 16 MiB problem: rotate over several operand sets so that no step finds
        # its inputs in L2 (the other workloads are far larger than L2 as they are)
        self.sets = C1_ROTATE if batch == 1 and 2 * (M + N) * K * self.bits // 8 < (64 << 20) else 1
        self.step_index = 0
        self._alloc()

    # -- seeded synthetic inputs, generated on the device item by item
    def _gen(self, rows, seed):
        torch, K = self.torch, self.K
        B = self.B * self.sets
        g = torch.Generator(device=self.device)
        g.manual_seed(seed)
        il = self.layout == "interleaved"
        if self.layout == "bytes":
            out = torch.empty((B, 2, rows, K), dtype=torch.uint8, device=self.device)
            for b in range(B):
                out[b] = torch.randint(0, 2, (2, rows, K), dtype=torch.uint8, device=self.device,
                                       generator=g)
            return out
        tdt = _torch_dtype(torch, self.dtype)
        shape = (B, rows, K, 2) if il else (B, 2, rows, K)
        out = torch.empty(shape, dtype=tdt, device=self.device)
        for b in range(B):
            if self.dtype in ("e4m3", "e5m2"):
                fmax = 448.0 if self.dtype == "e4m3" else 57344.0
                x = torch.randn(shape[1:], device=self.device, generator=g).clamp_(-4, 4)
                x.mul_(0.5 * fmax / 4)
            elif self.name.startswith("c5") or self.name.startswith("c1"):
                x = torch.rand(shape[1:], device=self.device, generator=g).mul_(2).sub_(1)
            else:
                x = torch.randn(shape[1:], device=self.device, generator=g).mul_(1 / math.sqrt(K))
            out[b] = x.to(tdt)
            del x
        return out

    def _alloc(self):
        torch, capi = self.torch, self.capi
        rank_seed = 0xCC61B + 17 * int(os.environ.get("RANK", "0"))
        self.a_in = self._gen(self.M, rank_seed + 1)
        self.b_in = self._gen(self.N, rank_seed + 2)
        out_dt = torch.int32 if self.type_out == TYPE_CODE["INT32"] else torch.float32
        self.c = torch.empty((self.B * self.sets, 2, self.M, self.N), dtype=out_dt,
                             device=self.device)
        in_axis = capi.INTERLEAVED if self.layout == "interleaved" else capi.PLANAR
        self.pipe = capi.Pipeline(self.B, self.M, self.N, self.K, self.type_in, self.type_out,
                                  variant=self.variant, input_complex_axis=in_axis)
        self.launches_per_step = self.pipe.launches
        self.pipe.set_overlap(False)
        self.plain_launches = self.pipe.launches  # transposes in front, one GEMM launch
        self.pipe.set_overlap(True)
        self.item_a = self.a_in[0].numel() * self.a_in.element_size()
        self.item_b = self.b_in[0].numel() * self.b_in.element_size()
        self.item_c = self.c[0].numel() * 4

    def hbm_bytes(self):
        n = sum(t.numel() * t.element_size() for t in (self.a_in, self.b_in, self.c))
        return n + self.pipe.scratch_bytes

    def describe_step(self):
        if self.layout == "bytes":
            return "byte samples -> operand expansion + GEMM, %d launches" % self.launches_per_step
        if self.variant == self.capi.OPT:
            if self.launches_per_step > self.plain_launches:
                return ("transpose A, B + GEMM in %d batch chunks, the transposes of later chunks "
                        "beside the GEMM of earlier ones; the roofline's GEMM time comes from "
                        "extra steps with the plain chain" % (self.launches_per_step // 3))
            return "transpose A, B + GEMM"
        return "GEMM"

    # -- one pass through the library's Pipeline; gemm_events = (begin, end) torch events
    def step(self, stream_handle: int, gemm_events=None):
        s = self.step_index % self.sets
        self.step_index += 1
        if gemm_events is not None:
            self.pipe.set_gemm_events(gemm_events[0].cuda_event, gemm_events[1].cuda_event)
        self.pipe.run(self.a_in.data_ptr() + s * self.B * self.item_a,
                      self.b_in.data_ptr() + s * self.B * self.item_b,
                      self.c.data_ptr() + s * self.B * self.item_c, stream_handle)
        if gemm_events is not None:
            self.pipe.set_gemm_events(None, None)

    # -- sampled parity check against float64 dot products of the same stored inputs
    def spot_check(self, samples=48, c=None):
        torch = self.torch
        c = self.c if c is None else c
        g = torch.Generator(device="cpu")
        g.manual_seed(1234)
        worst = 0.0
        K = self.K
        for _ in range(samples):
            b = int(torch.randint(0, self.B, (1,), generator=g))
            m = int(torch.randint(0, self.M, (1,), generator=g))
            n = int(torch.randint(0, self.N, (1,), generator=g))
            if self.layout == "interleaved":
                ar, ai = self.a_in[b, m, :, 0], self.a_in[b, m, :, 1]
                br, bi = self.b_in[b, n, :, 0], self.b_in[b, n, :, 1]
            else:
                ar, ai = self.a_in[b, 0, m], self.a_in[b, 1, m]
                br, bi = self.b_in[b, 0, n], self.b_in[b, 1, n]
            ar, ai, br, bi = (x.to(torch.float32).to(torch.float64) for x in (ar, ai, br, bi))
            if self.layout == "bytes":
                ar, ai, br, bi = (2 * x - 1 for x in (ar, ai, br, bi))
            elif self.dtype == "tf32":
                mask = lambda x: (x.to(torch.float32).view(torch.int32) & -8192).view(
                    torch.float32).to(torch.float64)
                ar, ai, br, bi = (mask(x) for x in (ar, ai, br, bi))
            re = float((ar * br).sum() - (ai * bi).sum())
            im = float((ar * bi).sum() + (ai * br).sum())
            s_re = float((ar.abs() * br.abs()).sum() + (ai.abs() * bi.abs()).sum())
            s_im = float((ar.abs() * bi.abs()).sum() + (ai.abs() * br.abs()).sum())
            got_re, got_im = float(c[b, 0, m, n]), float(c[b, 1, m, n])
            if self.type_in == TYPE_CODE["INT1"]:
                if got_re != re or got_im != im:
                    return {"samples": samples, "ok": False, "worst_err_over_tol": float("inf")}
                continue
            for got, want, s in ((got_re, re, s_re), (got_im, im, s_im)):
                # the library's stated gate: random-walk rounding + truncation bias of the
                # tensor core's adder (one MMA instruction per 32 bytes of K) + final rounding
                steps = 2.0 * K * self.bits / 256.0
                tol = (4.0 * math.sqrt(2 * K) * 2.0 ** -24 * s +
                       (steps + 1.0) * 2.0 ** -23 * abs(want) + 1e-30)
                worst = max(worst, abs(got - want) / tol)
        return {"samples": samples, "ok": worst <= 1.0, "worst_err_over_tol": worst,
                "gate": "4*sqrt(2K)*2^-24*S + (2K/k_mma + 1)*2^-23*|c| (exact for 1-bit)"}

    def _planes_f64(self, t, b):
        """(re, im) float64 planes [rows][K] of batch item b of an input tensor, as the GEMM sees
        them (1-bit: +-1; tf32: low 13 mantissa bits ignored)."""
        torch = self.torch
        if self.layout == "interleaved":
            re, im = t[b, :, :, 0], t[b, :, :, 1]
        else:
            re, im = t[b, 0], t[b, 1]
        re, im = re.to(torch.float32), im.to(torch.float32)
        if self.layout == "bytes":
            re, im = 2 * re - 1, 2 * im - 1
        elif self.dtype == "tf32":
            re = (re.view(torch.int32) & -8192).view(torch.float32)
            im = (im.view(torch.int32) & -8192).view(torch.float32)
        return re.to(torch.float64), im.to(torch.float64)

    def freivalds(self, max_items=4):
        """Whole-matrix check of up to max_items batch items: C x against A (B^T x) in float64 for
        a random complex vector x with small integer parts.  Every element of C enters the
        product, so a wrong tile, edge or plane shows up.  Allowed residual of row m: the
        per-element gate in its statistical form, 4 sqrt(2K) 2^-24 S(m, n), added in quadrature
        over n with weights |x_n|, with S(m, n) bounded by the product of the row norms of |A|
        and |B| (exact equality for 1-bit)."""
        torch = self.torch
        g = torch.Generator(device=self.device)
        g.manual_seed(4321)
        B, N, K = self.B, self.N, self.K
        items = sorted({0, B - 1, B // 2, B // 3})[:max_items]
        worst = 0.0
        for b in items:
            xr = torch.randint(-2, 3, (N,), generator=g, device=self.device).to(torch.float64)
            xi = torch.randint(-2, 3, (N,), generator=g, device=self.device).to(torch.float64)
            br, bi = self._planes_f64(self.b_in, b)
            wr = br.T @ xr - bi.T @ xi
            wi = br.T @ xi + bi.T @ xr
            b_norm = torch.linalg.vector_norm(br.abs() + bi.abs(), dim=1)
            spread = torch.sqrt((((xr.abs() + xi.abs()) * b_norm) ** 2).sum())
            del br, bi
            ar, ai = self._planes_f64(self.a_in, b)
            want_re = ar @ wr - ai @ wi
            want_im = ar @ wi + ai @ wr
            a_norm = torch.linalg.vector_norm(ar.abs() + ai.abs(), dim=1)
            del ar, ai
            cr, ci = self.c[b, 0].to(torch.float64), self.c[b, 1].to(torch.float64)
            got_re = cr @ xr - ci @ xi
            got_im = cr @ xi + ci @ xr
            del cr, ci
            err = torch.maximum((got_re - want_re).abs(), (got_im - want_im).abs())
            if self.type_in == TYPE_CODE["INT1"]:
                if float(err.max()) != 0.0:
                    return {"items": items, "ok": False, "worst_err_over_tol": float("inf")}
                continue
            tol = 4.0 * math.sqrt(2 * K) * 2.0 ** -24 * a_norm * spread + 1e-30
            worst = max(worst, float((err / tol).max()))
        return {"items": items, "ok": worst <= 1.0, "worst_err_over_tol": worst}

    # -- the reference's own GPU kernel on the first batch items of the same inputs
    def reference_gpu(self, stream_handle: int):
        """Runs the reference project's legacy WMMA / mma.sync kernel (compiled unmodified for
        sm_100a, one cubin per workload slice) on the first batch items of this workload's
        operands, compares its C with this library's for those items and times it.  Reported
        baseline and second checker only."""
        torch, capi = self.torch, self.capi
        try:
            import reference_gpu as rg
        except ImportError:
            return {"unavailable": "tests/reference_gpu.py not importable"}
        case = REFERENCE_GPU_CASE.get(self.name)
        if not rg.available() or case not in rg.manifest():
            return {"unavailable": "the reference's GPU kernels were not compiled "
                                   "(oracle/build_reference_gpu.py needs the reference checkout)"}
        info = rg.manifest()[case]
        nb = min(info["B"], self.B)
        if nb != info["B"]:
            return {"unavailable": "this rank holds fewer than %d batch items" % info["B"]}
        M, N, K = self.M, self.N, self.K
        a, b = self.a_in[:nb], self.b_in[:nb]
        bits, in_axis = self.bits, capi.PLANAR
        if self.layout == "interleaved":
            in_axis = capi.INTERLEAVED
        if self.layout == "bytes":  # the reference packs first (src/pipeline/Pipeline.cpp:108-112)
            pa = torch.empty(a.numel() // 8, dtype=torch.uint8, device=self.device)
            pb = torch.empty(b.numel() // 8, dtype=torch.uint8, device=self.device)
            capi.pack(a.numel(), capi.FORWARD, capi.PLANAR, a.data_ptr(), pa.data_ptr(),
                      stream_handle)
            capi.pack(b.numel(), capi.FORWARD, capi.PLANAR, b.data_ptr(), pb.data_ptr(),
                      stream_handle)
            a, b = pa, pb
        if info["variant"] == "opt":  # the reference kernel's own tile contract
            def tiled(x, rows, blk):
                rt, kt = -(-rows // blk), -(-K // info["k_chunk"])
                out = torch.zeros(nb * rt * kt * 2 * blk * info["k_chunk"] * bits // 8,
                                  dtype=torch.uint8, device=self.device)
                capi.transpose(nb, rows, K, blk, info["k_chunk"], bits, in_axis, x.data_ptr(),
                               out.data_ptr(), stream_handle)
                return out
            a, b = tiled(a, M, info["m_blk"]), tiled(b, N, info["n_blk"])
        elif in_axis != capi.PLANAR:
            return {"unavailable": "the reference's basic kernel reads planar input only"}
        c_ref = torch.zeros((nb, 2, M, N), dtype=self.c.dtype, device=self.device)

        def launch():
            rg.launch(case, c_ref.data_ptr(), a.data_ptr(), b.data_ptr(), stream_handle)

        launch()
        torch.cuda.synchronize()
        times = []
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            launch()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        ms = float(np.mean(times))
        ours = self.c[:nb]
        if self.type_in == TYPE_CODE["INT1"]:
            agrees = bool(torch.equal(ours, c_ref))
            rule = "identical"
        else:
            eps = {"f16": 2.0 ** -10, "bf16": 2.0 ** -7, "tf32": 2.0 ** -10, "e4m3": 0.125,
                   "e5m2": 0.25}[self.dtype]
            rel = (ours - c_ref).abs() / (ours.abs() + c_ref.abs() + 1.0)
            agrees = bool(float(rel.max()) <= 10.0 * eps)
            rule = "|x-y|/(|x|+|y|+1) <= 10 eps(Tin), the reference's test/gemm/fpequals.h rule"
        ops = 8.0 * M * N * K * nb
        return {"kernel": info["entry"] + " (reference kernels/, sm_100a cubin)", "batch": nb,
                "ms": ms, "tops": ops / ms / 1e9, "agrees_with_this_library": agrees,
                "rule": rule}


# --------------------------------------------------------------------------- end-to-end pass

class HostRun:
    """The same pass with HOST operands through the library's own host-memory call
    (ccglib_b200_pipeline_run_host, the counterpart of the reference's Pipeline::Run(HostMemory)):
    whole A, B and C in pinned host memory, filled from the seeded device inputs."""

    def __init__(self, wl: Workload):
        torch = wl.torch
        self.wl = wl
        t0 = time.perf_counter()
        nbytes = lambda t: wl.B * t[0].numel() * t.element_size()
        self.h_a = torch.empty(nbytes(wl.a_in), dtype=torch.uint8, pin_memory=True)
        self.h_b = torch.empty(nbytes(wl.b_in), dtype=torch.uint8, pin_memory=True)
        self.h_c = torch.empty(nbytes(wl.c), dtype=torch.uint8, pin_memory=True)
        self.h_a.copy_(wl.a_in[:wl.B].reshape(-1).view(torch.uint8))
        self.h_b.copy_(wl.b_in[:wl.B].reshape(-1).view(torch.uint8))
        self.h_c.zero_()
        torch.cuda.synchronize()
        self.setup_s = time.perf_counter() - t0
        self.h2d_bytes = self.h_a.numel() + self.h_b.numel()
        self.d2h_bytes = self.h_c.numel()

    def step(self, stream_handle):
        self.wl.pipe.run_host(self.h_a.data_ptr(), self.h_b.data_ptr(), self.h_c.data_ptr(),
                              stream_handle)

    def time_steps(self, steps, warmup, stream_handle):
        torch = self.wl.torch
        for _ in range(warmup):
            self.step(stream_handle)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            self.step(stream_handle)  # blocks until C is complete in host memory
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / steps

    def check(self):
        """The C that came back to host memory against the device-resident C of the device-timed
        steps (same kernels, same inputs: identical), first and last batch item in full, and
        against float64 dot products on sampled elements."""
        torch, wl = self.wl.torch, self.wl
        item = wl.item_c
        same = True
        for b in sorted({0, wl.B - 1}):
            back = self.h_c[b * item:(b + 1) * item].to(wl.device)
            same = same and bool(torch.equal(back, wl.c[b].reshape(-1).view(torch.uint8)))
        h_view = self.h_c.view(wl.c.dtype).reshape(wl.B, 2, wl.M, wl.N)
        spot = wl.spot_check(samples=16, c=h_view)
        return {"host_c_equals_device_c": same, "sampled_fp64": spot["ok"],
                "ok": bool(same and spot["ok"])}


# --------------------------------------------------------------------------- main arms

def run_reference_arm(args, name):
    dtype, tin, tout, B, M, N, K, variant, layout = WORKLOADS[name]
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals = []
    base = None
    for i in range(args.warmup + args.steps):
        base = cpu_baseline(tin, tout, K, target_s=min(12.0, 90.0 / (args.warmup + args.steps)))
        if i >= args.warmup:
            vals.append(base)
    value = float(np.mean([v["value"] for v in vals]))
    secs = float(np.mean([v["seconds"] for v in vals]))
    line = {
        "impl": "reference", "metric": "complex_tops", "value": value, "unit": "TOPS",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": secs * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": dtype, "data": "synthetic",
        "config": {"workload": name, "batch": B, "M": M, "N": N, "K": K, "variant": variant,
                   "input": layout, "note": "CPU reference GEMM timed on a bounded sample: "
                   + base["sample"]},
        "cpu_baseline": {"value": value, "unit": "TOPS", "cores": base["cores"],
                         "kind": base["kind"], "sample": base["sample"]},
        "e2e": {"value": value, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def roofline_of(name, dtype, M, N, K, bits, items, gemm_ms, peaks):
    scale = NOMINAL_TFLOPS[dtype] / NOMINAL_TFLOPS["bf16"]
    peak = peaks["bf16_tflops_sustained"] * scale
    achieved = 8.0 * M * N * K * items / (gemm_ms * 1e-3) / 1e12
    r = {
        "bound": "tensor", "kernel": "cgemm_pair_kernel" if dtype == "int1" else
        "cgemm_tcgen05_kernel", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
        "frac": achieved / peak,
        "traffic": (NCU_DRAM_BYTES_PER_ITEM[name] * items
                    if name in NCU_DRAM_BYTES_PER_ITEM else None),
        "traffic_source": ("single-launch ncu capture of a small case of the GEMM kernel, scaled "
                           "by the batch" if name in NCU_DRAM_BYTES_PER_ITEM else
                           "no ncu capture of this workload's kernel is wired in"),
        "algorithmic_bytes": items * (2.0 * (M + N) * K * bits / 8 + 2.0 * M * N * 4),
        "peak_source": "%s sustained bf16 GEMM x %.2g (nominal dtype rate ratio%s)" % (
            peaks["source"], scale,
            "; a proxy: the 4-bit pipe is not in MEASURED_PEAKS, quote frac_of_nominal"
            if dtype == "int1" else ""),
        "frac_of_burst": achieved / (peaks["bf16_tflops"] * scale),
        "frac_of_nominal": achieved / NOMINAL_TFLOPS[dtype],
        "gemm_ms_per_launch": gemm_ms,
    }
    # the other roof, for shapes near the ridge (config 5): algorithmic bytes / time
    r["hbm_gbs_achieved"] = r["algorithmic_bytes"] / (gemm_ms * 1e-3) / 1e9
    r["hbm_frac"] = r["hbm_gbs_achieved"] / peaks["hbm_gbs"]
    if r["hbm_frac"] > r["frac"]:
        r.update(bound="hbm", achieved=r["hbm_gbs_achieved"], peak=peaks["hbm_gbs"], unit="GB/s",
                 frac=r["hbm_frac"], tensor_tflops_achieved=achieved, tensor_frac=achieved / peak)
    return r


def measure_device(wl, steps, warmup, sampler, dist, world):
    """Warm-up, then `steps` timed steps between CUDA events on the launch stream; returns
    (ms per step, GEMM ms per launch, clocks), the times as max over ranks.  The GEMM stage is
    timed by an event pair per step.  Where the Pipeline runs its transposes beside the GEMM
    (several batch chunks), the stage of the timed steps is not one kernel alone, so the
    roofline's GEMM time is taken in a few extra steps right after the timed region, with the
    plain chain (transposes in front, one GEMM launch)."""
    torch, capi = wl.torch, wl.capi
    stream = torch.cuda.current_stream()
    handle = int(stream.cuda_stream)
    for _ in range(max(warmup, 3)):
        wl.step(handle)
    torch.cuda.synchronize()
    status = capi.device_status()
    if status:
        raise SystemExit("device status word 0x%x after warm-up" % status)
    overlapped = wl.pipe.launches > wl.plain_launches

    def event_pairs(n):
        pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                 for _ in range(n)]
        for a, b in pairs:  # torch creates the CUDA event at its first record: the handles must exist
            a.record()
            b.record()
        return pairs

    gemm_ev = event_pairs(min(steps, 200))
    extra_ev = event_pairs(max(3, min(steps // 2, 10))) if overlapped else []
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    if sampler is not None:
        sampler.start()
        time.sleep(0.25)
    start.record()
    for i in range(steps):
        wl.step(handle, gemm_ev[i] if i < len(gemm_ev) and not overlapped else None)
    stop.record()
    if overlapped:  # same thermal and clock state: straight after the timed steps
        wl.pipe.set_overlap(False)
        for pair in extra_ev:
            wl.step(handle, pair)
        wl.pipe.set_overlap(True)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop() if sampler is not None else None
    ms_total = start.elapsed_time(stop)
    gemm_ms = float(np.mean([a.elapsed_time(b) for a, b in (extra_ev if overlapped else gemm_ev)]))
    status = capi.device_status()
    if status:
        raise SystemExit("device status word 0x%x in the timed region" % status)
    t = torch.tensor([ms_total, gemm_ms], dtype=torch.float64, device=wl.device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0]) / steps, float(t[1]), clocks


def steps_for(wl, seconds, dist, world):
    """Steps that fill about `seconds` of device time (same count on every rank)."""
    torch = wl.torch
    handle = int(torch.cuda.current_stream().cuda_stream)
    for _ in range(3):
        wl.step(handle)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        wl.step(handle)
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / 3.0], dtype=torch.float64, device=wl.device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return int(max(5, min(100000, math.ceil(seconds * 1e3 / max(float(t[0]), 1e-3)))))


def run_ours(args, name):
    import torch
    import torch.distributed as dist

    from ccglib_b200 import capi, sharding

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    capi.lib()  # fail loudly if the CUDA library is missing
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    peaks = measured_peaks()
    handle = int(torch.cuda.current_stream().cuda_stream)

    def config_of(wname, B_total, share, wl, hbm_gb):
        dtype, tin, tout, _, M, N, K, variant, layout = WORKLOADS[wname]
        return {"workload": wname, "batch": B_total, "batch_per_gpu": share, "M": M, "N": N,
                "K": K, "variant": variant, "input": layout, "step": wl.describe_step(),
                "l2": ("operands rotate over %d sets (%.0f MB) larger than L2" % (
                    wl.sets, hbm_gb * 1e3) if wl.sets > 1 else
                    "inputs larger than L2 (%.1f GB resident per GPU)" % hbm_gb),
                "parallelism": "batch split over %d GPU(s), no collective" % world}

    # ---- headline workload
    dtype, tin, tout, B_total, M, N, K, variant, layout = WORKLOADS[name]
    if args.batch:
        B_total = args.batch
    # batch items are independent GEMMs: rank r takes a contiguous share, no collective needed
    share = sharding.batch_shares(B_total, world)
    B = share[rank]
    if B == 0:
        raise SystemExit("batch %d cannot be split over %d ranks" % (B_total, world))
    wl = Workload(name, B, device)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    ms_step, gemm_ms, clocks = measure_device(wl, args.steps, args.warmup, sampler, dist, world)
    check = wl.spot_check()
    check["freivalds"] = wl.freivalds()
    check["ok"] = bool(check["ok"] and check["freivalds"]["ok"])
    ref_gpu = wl.reference_gpu(handle) if rank == 0 and not args.no_reference_gpu else None
    hbm_gb = wl.hbm_bytes() / 1e9
    launches = wl.launches_per_step * args.steps
    total_flops = 8.0 * M * N * K * B_total
    value = total_flops / (ms_step * 1e-3) / 1e12
    roofline = roofline_of(name, dtype, M, N, K, wl.bits, share[0], gemm_ms, peaks)
    config = config_of(name, B_total, share[0], wl, hbm_gb)

    # ---- end to end with host operands (every rank runs it; the slowest rank's time counts)
    e2e = None
    if not args.no_e2e:
        hr = HostRun(wl)
        if world > 1:
            dist.barrier()
        sec = hr.time_steps(max(1, args.e2e_steps), 1, handle)
        te = torch.tensor([sec], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e = {"value": total_flops / float(te[0]) / 1e12, "unit": "TOPS",
               "h2d_bytes_per_step": hr.h2d_bytes * world, "d2h_bytes_per_step": hr.d2h_bytes * world,
               "ms_per_step": float(te[0]) * 1e3, "steps": max(1, args.e2e_steps), "warmup": 1,
               "slice_items": wl.pipe.host_slice,
               "call": "ccglib_b200_pipeline_run_host (ccglib::pipeline::Pipeline::Run on host "
                       "memory): whole A, B, C pinned on the host, sliced and double-buffered "
                       "inside the library",
               "host_setup_s": hr.setup_s, "check": hr.check()}
        status = capi.device_status()
        if status:
            raise SystemExit("device status word 0x%x in the end-to-end pass" % status)
        del hr
    del wl
    torch.cuda.empty_cache()

    # ---- the other workloads of the baseline, each device-timed for about two seconds
    per_workload = None
    if args.per_workload and args.workload is None:
        per_workload = {}
        for other in sorted(WORKLOADS):
            if other == name:
                continue
            o_dtype, o_tin, o_tout, o_B, o_M, o_N, o_K, o_variant, o_layout = WORKLOADS[other]
            if o_B < world:
                if rank == 0:
                    per_workload[other] = {"skipped": "batch %d cannot be split over %d GPUs "
                                                      "(replicas only)" % (o_B, world)}
                continue
            o_share = sharding.batch_shares(o_B, world)
            owl = Workload(other, o_share[rank], device)
            o_steps = steps_for(owl, args.per_workload_seconds, dist, world)
            o_sampler = ClockSampler(local_rank) if rank == 0 else None
            o_ms, o_gemm_ms, o_clocks = measure_device(owl, o_steps, 3, o_sampler, dist, world)
            o_check = owl.spot_check()
            o_check["freivalds"] = owl.freivalds()
            o_check["ok"] = bool(o_check["ok"] and o_check["freivalds"]["ok"])
            ok_all = torch.tensor([1.0 if o_check["ok"] else 0.0], device=device)
            if world > 1:
                dist.all_reduce(ok_all, op=dist.ReduceOp.MIN)
            o_check["ok_on_every_rank"] = bool(float(ok_all[0]) == 1.0)
            if rank == 0:
                o_hbm = owl.hbm_bytes() / 1e9
                per_workload[other] = {
                    "value": 8.0 * o_M * o_N * o_K * o_B / (o_ms * 1e-3) / 1e12, "unit": "TOPS",
                    "dtype": o_dtype, "ms_per_step": o_ms, "steps": o_steps, "warmup": 3,
                    "config": config_of(other, o_B, o_share[0], owl, o_hbm),
                    "roofline": roofline_of(other, o_dtype, o_M, o_N, o_K, owl.bits, o_share[0],
                                            o_gemm_ms, peaks),
                    "gpu_launches": owl.launches_per_step * o_steps,
                    "parity": o_check, "clocks": o_clocks,
                    "reference_gpu": (None if args.no_reference_gpu
                                      else owl.reference_gpu(handle)),
                }
            del owl
            torch.cuda.empty_cache()

    if rank == 0:
        base = None if args.no_cpu_baseline or world > 1 else cpu_baseline(tin, tout, K)
        line = {
            "metric": "complex_tops", "value": value, "unit": "TOPS", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": dtype,
            "data": "synthetic", "config": config,
            "roofline": roofline, "cpu_baseline": base, "e2e": e2e, "gpu_launches": launches,
            "clocks": clocks, "parity": check, "reference_gpu": ref_gpu,
            "per_workload": per_workload,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS),
                    help="run this workload alone (default: the headline workload plus a "
                         "per_workload block for all the others)")
    ap.add_argument("--batch", type=int, default=0, help="override the batch size (experiments)")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--per-workload-seconds", type=float, default=2.0)
    ap.add_argument("--no-per-workload", dest="per_workload", action="store_false")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-reference-gpu", action="store_true")
    args = ap.parse_args()
    name = args.workload or DEFAULT_WORKLOAD
    if args.impl == "reference":
        run_reference_arm(args, name)
    else:
        run_ours(args, name)


if __name__ == "__main__":
    main()
