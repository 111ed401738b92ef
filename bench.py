"""Benchmark of the complex-GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one pass of the hot path over the whole (per-rank share of the) workload.  The
default workload is the optimized fp16 -> fp32 complex GEMM on interleaved input, batch 64,
M = N = K = 8192: Transpose(A), Transpose(B), GEMM, all enqueued on one stream through the C ABI.
Metric: complex TOPS = 8*M*N*K*batch / time (the reference's benchmark/benchmark_gemm.cpp:79-82).

* `value`    inputs resident in HBM, CUDA-event time of K steps, max over ranks.
* `e2e`      the same pass with HOST buffers: pinned host -> device copies of A and B and the
             device -> host copy of C inside the timed region (double-buffered batch slices).
* `roofline` the GEMM kernel alone: 8*M*N*K*batch flops per launch / its CUDA-event duration,
             against the measured tensor peak in MEASURED_PEAKS.json.
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
    # 1-bit: Packing, then the GEMM on the packed [batch][2][rows][K/32] words; the GEMM re-stages
    # 1-bit operands itself, so the Pipeline does not tile them first
    "c3_int1_4096_k65536_b32": ("int1", "INT1", "INT32", 32, 4096, 4096, 65536, "basic", "bytes"),
    "c4_e4m3_4096_k16384_b32": ("e4m3", "E4M3", "F32", 32, 4096, 4096, 16384, "opt", "planar"),
    "c4_e5m2_4096_k16384_b32": ("e5m2", "E5M2", "F32", 32, 4096, 4096, 16384, "opt", "planar"),
    "c5_bf16_256x2048x512_b4096": ("bf16", "BF16", "F32", 4096, 256, 2048, 512, "basic", "planar"),
    "c5_tf32_256x2048x512_b4096": ("tf32", "F32", "F32", 4096, 256, 2048, 512, "basic", "planar"),
}
DEFAULT_WORKLOAD = "c2_f16_opt_8192_b64"

# value-type codes of the C ABI (= the reference's ValueType ordinals) and their widths in bits
TYPE_CODE = {"INT1": 0, "INT32": 1, "BF16": 2, "E4M3": 3, "E5M2": 4, "F16": 5, "F32": 6}
TYPE_BITS = {0: 1, 1: 32, 2: 16, 3: 8, 4: 8, 5: 16, 6: 32}

# DRAM bytes (read + write) of one GEMM launch per batch item, from the ncu capture summarised in
# profiles/cgemm_tcgen05_f16_opt_8192_batch2_ncu_full.md (6.79 GB for 2 items; items are walked
# one after another, so traffic grows in proportion to the batch).
NCU_DRAM_BYTES_PER_ITEM = {"c2_f16_opt_8192_b64": 3.39e9}


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

def cpu_baseline(type_in_name: str, type_out_name: str, K: int, target_s: float = 12.0) -> dict:
    """Times the reference's own CPU GEMM (or the C restatement) on a bounded sample: one batch
    item of the workload's dtype and K with M = N chosen so the run takes about target_s."""
    import oracle_util as ou

    type_in = getattr(ou, type_in_name)
    type_out = getattr(ou, type_out_name)
    ref = ou.load_reference()
    kind = "reference" if ref is not None else "port"
    cores = os.cpu_count() or 1
    os.environ.setdefault("OMP_NUM_THREADS", str(cores))
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
            "sample": "1 batch item, M=N=%d, K=%d, %s->%s, %.1f s" % (
                mn, K, type_in_name.lower(), type_out_name.lower(), t),
            "seconds": t}


# --------------------------------------------------------------------------- device workload

class Workload:
    """Device-resident buffers and the enqueue function of one pass of the hot path."""

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
        self.flops = 8.0 * M * N * K * batch
        self.launches_per_step = 1
        self.m_blk, self.n_blk, self.k_c = capi.gemm_dims(self.type_in, self.type_out, self.variant)
        self._alloc()

    # -- allocation and seeded synthetic inputs (generated on the device, item by item)
    def _gen(self, rows, seed):
        torch, B, K = self.torch, self.B, self.K
        g = torch.Generator(device=self.device)
        g.manual_seed(seed)
        il = self.layout == "interleaved"
        if self.layout == "bytes":
            out = torch.empty((B, 2, rows, K), dtype=torch.uint8, device=self.device)
            for b in range(B):
                out[b] = torch.randint(0, 2, (2, rows, K), dtype=torch.uint8, device=self.device,
                                       generator=g)
            return out
        tdt = {"f16": torch.float16, "bf16": torch.bfloat16, "tf32": torch.float32,
               "e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}[self.dtype]
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

    def _tiled_bytes(self, rows, blk):
        rt = -(-rows // blk)
        kt = -(-self.K // self.k_c)
        return self.B * rt * kt * 2 * blk * self.k_c * self.bits // 8

    def _alloc(self):
        torch, capi = self.torch, self.capi
        rank_seed = 0xCC61B + 17 * int(os.environ.get("RANK", "0"))
        self.a_in = self._gen(self.M, rank_seed + 1)
        self.b_in = self._gen(self.N, rank_seed + 2)
        self.a_gemm, self.b_gemm = self.a_in, self.b_in
        if self.layout == "bytes":
            self.a_packed = torch.empty(self.a_in.numel() // 8, dtype=torch.uint8,
                                        device=self.device)
            self.b_packed = torch.empty(self.b_in.numel() // 8, dtype=torch.uint8,
                                        device=self.device)
            self.a_gemm, self.b_gemm = self.a_packed, self.b_packed
            self.launches_per_step += 2
        if self.variant == capi.OPT:
            self.a_tiled = torch.empty(self._tiled_bytes(self.M, self.m_blk), dtype=torch.uint8,
                                       device=self.device)
            self.b_tiled = torch.empty(self._tiled_bytes(self.N, self.n_blk), dtype=torch.uint8,
                                       device=self.device)
            self.a_gemm, self.b_gemm = self.a_tiled, self.b_tiled
            self.launches_per_step += 2
        out_dt = torch.int32 if self.type_out == TYPE_CODE["INT32"] else torch.float32
        self.c = torch.empty((self.B, 2, self.M, self.N), dtype=out_dt, device=self.device)
        self.plan = capi.GemmPlan(self.B, self.M, self.N, self.K, self.type_in, self.type_out,
                                  variant=self.variant)
        self.launches_per_step += self.plan.launches - 1

    def hbm_bytes(self):
        n = sum(t.numel() * t.element_size() for t in (self.a_in, self.b_in, self.c))
        for name in ("a_packed", "b_packed", "a_tiled", "b_tiled"):
            if hasattr(self, name):
                n += getattr(self, name).numel()
        return n + self.plan.scratch_bytes

    # -- one pass; returns (event before GEMM, event after GEMM) when asked
    def step(self, stream_handle: int, gemm_events=None):
        capi = self.capi
        a, b = self.a_in, self.b_in
        in_axis = capi.INTERLEAVED if self.layout == "interleaved" else capi.PLANAR
        if self.layout == "bytes":
            capi.pack(a.numel(), capi.FORWARD, capi.PLANAR, a.data_ptr(), self.a_packed.data_ptr(),
                      stream_handle)
            capi.pack(b.numel(), capi.FORWARD, capi.PLANAR, b.data_ptr(), self.b_packed.data_ptr(),
                      stream_handle)
            a, b = self.a_packed, self.b_packed
        if self.variant == capi.OPT:
            capi.transpose(self.B, self.M, self.K, self.m_blk, self.k_c, self.bits, in_axis,
                           a.data_ptr(), self.a_tiled.data_ptr(), stream_handle)
            capi.transpose(self.B, self.N, self.K, self.n_blk, self.k_c, self.bits, in_axis,
                           b.data_ptr(), self.b_tiled.data_ptr(), stream_handle)
        if gemm_events is not None:
            gemm_events[0].record()
        self.plan.run(self.a_gemm.data_ptr(), self.b_gemm.data_ptr(), self.c.data_ptr(),
                      stream_handle)
        if gemm_events is not None:
            gemm_events[1].record()

    # -- sampled parity check against float64 dot products of the same stored inputs
    def spot_check(self, samples=48):
        torch = self.torch
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
            got_re, got_im = float(self.c[b, 0, m, n]), float(self.c[b, 1, m, n])
            if self.type_in == TYPE_CODE["INT1"]:
                if got_re != re or got_im != im:
                    return {"samples": samples, "ok": False, "worst_err_over_tol": float("inf")}
                continue
            for got, want, s in ((got_re, re, s_re), (got_im, im, s_im)):
                tol = 2.0 * (2 * K + 2) * 2.0 ** -24 * s + 1e-30
                worst = max(worst, abs(got - want) / tol)
        return {"samples": samples, "ok": worst <= 1.0, "worst_err_over_tol": worst}


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


# --------------------------------------------------------------------------- end-to-end pass

class HostPipeline:
    """The same pass with HOST buffers: slices of the batch are copied from pinned host memory,
    transposed, multiplied and copied back, double-buffered over three streams so copies overlap
    compute.  Only built for workloads whose step is transpose + GEMM or GEMM alone."""

    def __init__(self, name: str, batch: int, device, slice_items: int):
        import torch

        from ccglib_b200 import capi

        self.torch, self.capi = torch, capi
        dtype, tin, tout, _, M, N, K, variant, layout = WORKLOADS[name]
        self.B, self.M, self.N, self.K = batch, M, N, K
        self.type_in, self.type_out = TYPE_CODE[tin], TYPE_CODE[tout]
        self.bits = TYPE_BITS[self.type_in]
        if slice_items <= 0:  # about 1 GiB of input per slice
            per_item = 2 * (M + N) * K * (8 if layout == "bytes" else self.bits) // 8
            slice_items = max(1, (1 << 30) // per_item)
        self.S = max(1, min(slice_items, batch))
        while batch % self.S:
            self.S -= 1
        self.variant = capi.OPT if variant == "opt" else capi.BASIC
        self.layout = layout
        self.packed = layout == "bytes"
        S = self.S
        in_bytes_a = S * 2 * M * K * (8 if self.packed else self.bits) // 8
        in_bytes_b = S * 2 * N * K * (8 if self.packed else self.bits) // 8
        c_bytes = S * 2 * M * N * 4
        self.h2d_bytes = (in_bytes_a + in_bytes_b) * (batch // S)
        self.d2h_bytes = c_bytes * (batch // S)
        u8 = torch.uint8
        g = torch.Generator()
        g.manual_seed(99)
        # host slices hold valid patterns of the input type (small fp16-like magnitudes / 0-1)
        self.h_a = torch.empty(in_bytes_a, dtype=u8).pin_memory()
        self.h_b = torch.empty(in_bytes_b, dtype=u8).pin_memory()
        self.h_c = torch.empty(c_bytes, dtype=u8).pin_memory()
        if self.packed:
            self.h_a.copy_(torch.randint(0, 2, (in_bytes_a,), dtype=u8, generator=g))
            self.h_b.copy_(torch.randint(0, 2, (in_bytes_b,), dtype=u8, generator=g))
        else:
            # byte 0x2c in every position decodes to a small finite value in f16/bf16/fp8/f32
            self.h_a.fill_(0x2C)
            self.h_b.fill_(0x2C)
        self.d_a = [torch.empty(in_bytes_a, dtype=u8, device=device) for _ in range(2)]
        self.d_b = [torch.empty(in_bytes_b, dtype=u8, device=device) for _ in range(2)]
        self.d_c = [torch.empty(c_bytes, dtype=u8, device=device) for _ in range(2)]
        self.m_blk, self.n_blk, self.k_c = capi.gemm_dims(self.type_in, self.type_out, self.variant)
        if self.packed:
            self.p_a = torch.empty(in_bytes_a // 8, dtype=u8, device=device)
            self.p_b = torch.empty(in_bytes_b // 8, dtype=u8, device=device)
        if self.variant == capi.OPT:
            tb = lambda rows, blk: (S * (-(-rows // blk)) * (-(-K // self.k_c)) * 2 * blk *
                                    self.k_c * self.bits // 8)
            self.t_a = torch.empty(tb(M, self.m_blk), dtype=u8, device=device)
            self.t_b = torch.empty(tb(N, self.n_blk), dtype=u8, device=device)
        self.plan = capi.GemmPlan(S, M, N, K, self.type_in, self.type_out, variant=self.variant)
        self.s_in, self.s_cmp, self.s_out = (torch.cuda.Stream(device=device) for _ in range(3))
        self.ev_in = [torch.cuda.Event() for _ in range(2)]
        self.ev_cmp = [torch.cuda.Event() for _ in range(2)]
        self.ev_out = [torch.cuda.Event() for _ in range(2)]

    def step(self):
        torch, capi = self.torch, self.capi
        S, M, N, K = self.S, self.M, self.N, self.K
        in_axis = capi.INTERLEAVED if self.layout == "interleaved" else capi.PLANAR
        for i in range(self.B // S):
            buf = i & 1
            with torch.cuda.stream(self.s_in):
                self.s_in.wait_event(self.ev_cmp[buf])
                self.d_a[buf].copy_(self.h_a, non_blocking=True)
                self.d_b[buf].copy_(self.h_b, non_blocking=True)
                self.ev_in[buf].record()
            with torch.cuda.stream(self.s_cmp):
                self.s_cmp.wait_event(self.ev_in[buf])
                self.s_cmp.wait_event(self.ev_out[buf])
                h = int(self.s_cmp.cuda_stream)
                a, b = self.d_a[buf], self.d_b[buf]
                if self.packed:
                    capi.pack(a.numel(), capi.FORWARD, capi.PLANAR, a.data_ptr(),
                              self.p_a.data_ptr(), h)
                    capi.pack(b.numel(), capi.FORWARD, capi.PLANAR, b.data_ptr(),
                              self.p_b.data_ptr(), h)
                    a, b = self.p_a, self.p_b
                if self.variant == capi.OPT:
                    capi.transpose(S, M, K, self.m_blk, self.k_c, self.bits, in_axis, a.data_ptr(),
                                   self.t_a.data_ptr(), h)
                    capi.transpose(S, N, K, self.n_blk, self.k_c, self.bits, in_axis, b.data_ptr(),
                                   self.t_b.data_ptr(), h)
                    a, b = self.t_a, self.t_b
                self.plan.run(a.data_ptr(), b.data_ptr(), self.d_c[buf].data_ptr(), h)
                self.ev_cmp[buf].record()
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_cmp[buf])
                self.h_c.copy_(self.d_c[buf], non_blocking=True)
                self.ev_out[buf].record()

    def time_steps(self, steps, warmup):
        torch = self.torch
        for _ in range(warmup):
            self.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            self.step()
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / steps


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


def run_ours(args, name):
    import torch
    import torch.distributed as dist

    from ccglib_b200 import capi

    dtype, tin, tout, B_total, M, N, K, variant, layout = WORKLOADS[name]
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
    if args.batch:
        B_total = args.batch
    # batch items are independent GEMMs: rank r takes a contiguous share, no collective needed
    from ccglib_b200 import sharding

    share = sharding.batch_shares(B_total, world)
    B = share[rank]
    if B == 0:
        raise SystemExit("batch %d cannot be split over %d ranks" % (B_total, world))

    wl = Workload(name, B, device)
    stream = torch.cuda.current_stream()
    handle = int(stream.cuda_stream)
    for _ in range(max(args.warmup, 3)):
        wl.step(handle)
    torch.cuda.synchronize()
    status = capi.device_status()
    if status:
        raise SystemExit("device status word 0x%x after warm-up" % status)

    sampler = ClockSampler(local_rank)
    gemm_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
               for _ in range(args.steps)]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    start.record()
    for i in range(args.steps):
        wl.step(handle, gemm_ev[i])
    stop.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms_total = start.elapsed_time(stop)
    gemm_ms = float(np.mean([a.elapsed_time(b) for a, b in gemm_ev]))
    status = capi.device_status()
    if status:
        raise SystemExit("device status word 0x%x in the timed region" % status)
    t = torch.tensor([ms_total, gemm_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t[0]) / args.steps
    gemm_ms_max = float(t[1])
    check = wl.spot_check()
    check["freivalds"] = wl.freivalds()
    check["ok"] = bool(check["ok"] and check["freivalds"]["ok"])
    wl_bits = wl.bits
    hbm_gb = wl.hbm_bytes() / 1e9
    launches = wl.launches_per_step * args.steps
    total_flops = 8.0 * M * N * K * B_total
    value = total_flops / (ms_step * 1e-3) / 1e12

    # ---- end to end with host buffers (all ranks run it, rank 0 reports the max time)
    e2e = None
    if not args.no_e2e:
        del wl
        torch.cuda.empty_cache()
        hp = HostPipeline(name, B, device, args.e2e_slice)
        if world > 1:
            dist.barrier()
        sec = hp.time_steps(max(1, args.e2e_steps), 1)
        te = torch.tensor([sec], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e = {"value": total_flops / float(te[0]) / 1e12, "unit": "TOPS",
               "h2d_bytes_per_step": hp.h2d_bytes * world, "d2h_bytes_per_step": hp.d2h_bytes * world,
               "ms_per_step": float(te[0]) * 1e3, "slice_items": hp.S}
        status = capi.device_status()
        if status:
            raise SystemExit("device status word 0x%x in the end-to-end pass" % status)
        del hp

    if rank == 0:
        peaks = measured_peaks()
        scale = NOMINAL_TFLOPS[dtype] / NOMINAL_TFLOPS["bf16"]
        peak = peaks["bf16_tflops_sustained"] * scale
        gemm_flops_rank = 8.0 * M * N * K * share[0]
        achieved = gemm_flops_rank / (gemm_ms_max * 1e-3) / 1e12
        roofline = {
            "bound": "tensor", "kernel": "cgemm_tcgen05_kernel", "achieved": achieved,
            "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
            "traffic": (NCU_DRAM_BYTES_PER_ITEM[name] * share[0]
                        if name in NCU_DRAM_BYTES_PER_ITEM else None),
            "algorithmic_bytes": share[0] * (2.0 * (M + N) * K * wl_bits / 8 + 2.0 * M * N * 4),
            "peak_source": "%s sustained bf16 GEMM x %.2g (dtype rate ratio)" % (
                peaks["source"], scale),
            "frac_of_burst": achieved / (peaks["bf16_tflops"] * scale),
            "frac_of_nominal": achieved / NOMINAL_TFLOPS[dtype],
            "gemm_ms_per_launch": gemm_ms_max,
        }
        # the other roof, for shapes near the ridge (config 5): algorithmic bytes / time
        roofline["hbm_gbs_achieved"] = roofline["algorithmic_bytes"] / (gemm_ms_max * 1e-3) / 1e9
        roofline["hbm_frac"] = roofline["hbm_gbs_achieved"] / peaks["hbm_gbs"]
        if roofline["hbm_frac"] > roofline["frac"]:
            roofline.update(bound="hbm", achieved=roofline["hbm_gbs_achieved"],
                            peak=peaks["hbm_gbs"], unit="GB/s", frac=roofline["hbm_frac"],
                            tensor_tflops_achieved=achieved, tensor_frac=achieved / peak)
        base = None if args.no_cpu_baseline or world > 1 else cpu_baseline(tin, tout, K)
        line = {
            "metric": "complex_tops", "value": value, "unit": "TOPS", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": dtype,
            "data": "synthetic",
            "config": {"workload": name, "batch": B_total, "batch_per_gpu": share[0], "M": M,
                       "N": N, "K": K, "variant": variant, "input": layout,
                       "step": ("transpose A, B + GEMM" if variant == "opt" else
                                "pack A, B + GEMM" if layout == "bytes" else "GEMM"),
                       "l2": "inputs larger than L2 (%.1f GB resident per GPU)" % hbm_gb,
                       "parallelism": "batch split over %d GPU(s), no collective" % world},
            "roofline": roofline, "cpu_baseline": base, "e2e": e2e, "gpu_launches": launches,
            "clocks": clocks, "parity": check,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=0, help="override the batch size (experiments)")
    ap.add_argument("--e2e-steps", type=int, default=2)
    ap.add_argument("--e2e-slice", type=int, default=0,
                    help="batch items per host slice (0: about 1 GiB of input)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args, args.workload)
    else:
        run_ours(args, args.workload)


if __name__ == "__main__":
    main()
