#!/usr/bin/env python
"""Benchmark of the quantized-GEMM path on B200 (and of the reference's CPU path).

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload NAME]

One "step" is one GEMM call of the workload.  The default workload is the
headline single-GPU configuration: MX fp8 `GemmMxE4M3`, M=N=K=4096, TN,
alpha=1, beta=0.5, E8M0 scales in [122,132], C ~ N(0,1).  With N > 1 ranks
(torchrun, one process per GPU) the output is sharded by row blocks: every rank
owns a 4096-row block of a (4096*N) x 4096 x 4096 problem and all of B (weak
scaling, no data-path collective).

Prints ONE JSON line (rank 0).  `value` is device-resident throughput (CUDA
events around K asynchronous calls, max over ranks); `e2e` is the same metric
through the synchronous C-ABI call with pinned HOST buffers, host<->device
copies included; `roofline` is the tensor-core kernel alone, timed live with
CUDA events on its stream; `cpu_baseline` is the reference's own CPU operator
(oracle/_ref, built from the unmodified reference headers) on the host cores.

The same line carries, beside the headline:
  * `suite` (N = 1): one record per configured workload (int8 / mxfp8 / mxfp4 GEMMs at the
    configured and the 8192^3 / 16384^3 shapes, the decode shapes), each with its call time
    back to back over rotating operand sets, its kernel time, its launch plan and a
    roofline against the measured and the nominal peak -- the table the reference's
    benchmark prints in one run (examples/01_benchmark.cc:204-343);
  * `sharded` (N > 1): the 16384^3 MX problems cut into output row blocks over the N
    ranks (B replicated), timed without and with the all-gather of D, each rank's block
    checked against the CPU oracle at sampled positions and, bit for bit, against
    rank 0's own single-GPU computation of the same rows.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# nominal per-GPU figures of a B200: dense int8 / fp8, dense fp4 (TOP/s), HBM3e (GB/s)
NOMINAL_PEAKS = {2.0: 4500.0, 4.0: 9000.0, "hbm_gbs": 8000.0}


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return d, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


# ---------------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------------
class Workload:
    """A GEMM configuration: host operand generation, argument construction,
    algorithmic work."""

    def __init__(self, name):
        from cpu_ops_b200 import _capi
        self.name = name
        self.kind = "mx"
        self.fmt = _capi.FMT_E4M3
        self.m = self.n = self.k = 4096
        self.alpha, self.beta = 1.0, 0.5
        self.scale_lo, self.scale_hi = 122, 132
        self.split_k = 0
        self.chain = None
        self.bound = "tensor"
        if name == "mxfp8_e4m3_4096":
            pass
        elif name == "int8_2048":
            self.kind, self.m, self.n, self.k = "int8", 2048, 2048, 2048
            self.alpha, self.beta, self.split_k = 1, 1, 1
        elif name == "int8_8192_chain":
            self.kind, self.m, self.n, self.k = "int8", 8192, 8192, 16384
            self.alpha, self.beta, self.chain = 1, 0, "bias_relu_clamp"
        elif name == "int8_8192":
            self.kind, self.m, self.n, self.k = "int8", 8192, 8192, 8192
            self.alpha, self.beta = 1, 0
        elif name in ("mxfp8_8192", "mxfp4_8192"):
            self.fmt = _capi.FMT_E4M3 if name == "mxfp8_8192" else _capi.FMT_E2M1
            self.m = self.n = self.k = 8192
            self.beta = 0.0
        elif name in ("mx_e5m2_16384", "mx_e2m1_16384"):
            self.fmt = _capi.FMT_E5M2 if "e5m2" in name else _capi.FMT_E2M1
            self.m = self.n = self.k = 16384
            self.beta, self.scale_lo, self.scale_hi = 0.0, 120, 134
        elif name.startswith("mxfp4_decode_m"):
            self.fmt = _capi.FMT_E2M1
            self.m, self.n, self.k = int(name.rsplit("m", 1)[1]), 14336, 4096
            self.beta, self.scale_lo, self.scale_hi = 0.0, 124, 130
            self.bound = "hbm"
        else:
            raise SystemExit(f"unknown workload {name}")

    # algorithmic work of one step for `rows` output rows
    def ops(self, rows=None):
        rows = self.m if rows is None else rows
        return 2.0 * rows * self.n * self.k

    def min_bytes(self, rows=None):
        from cpu_ops_b200 import workloads as W
        rows = self.m if rows is None else rows
        if self.kind == "int8":
            return W.gemm_min_bytes(rows, self.n, self.k, 1, 1, False, self.beta != 0,
                                    self.chain is not None)
        b = W.FMT_BYTES_PER_ELEM[self.fmt]
        return W.gemm_min_bytes(rows, self.n, self.k, b, b, True, self.beta != 0)

    def host_operands(self, seed, rows=None):
        """dict of flat numpy arrays for `rows` output rows (default: all)."""
        from cpu_ops_b200 import workloads as W
        rows = self.m if rows is None else rows
        if self.kind == "int8":
            P = W.int8_problem(rows, self.n, self.k, True, True, True, seed=seed)
            out = dict(A=P.A, B=P.B, C=P.C, D=np.zeros_like(P.C))
            if self.chain:
                out["bias"] = W.rng_for(seed, 9).integers(-(1 << 15), (1 << 15) + 1, size=self.n,
                                                          dtype=np.int32)
            return out
        P = W.mx_problem(self.fmt, rows, self.n, self.k, True, scale_lo=self.scale_lo,
                         scale_hi=self.scale_hi, seed=seed)
        return dict(A=P.A, SA=P.SA, B=P.B, SB=P.SB, C=P.C, D=np.zeros_like(P.C))

    def device_operands(self, dev, seed, rows=None):
        """The same operands generated on the device (torch's counter-based generator: the
        same seed gives the same bytes on every B200), for workloads whose host generation
        would dominate the run.  MX elements avoid NaN / Inf codes; C is only generated
        when beta != 0 (otherwise the never-read C argument aliases D)."""
        import torch
        from cpu_ops_b200 import _capi
        rows = self.m if rows is None else rows
        n, k = self.n, self.k
        g = torch.Generator(device=dev)
        g.manual_seed(int(seed))

        def raw(count):
            return torch.randint(0, 256, (count,), dtype=torch.uint8, device=dev, generator=g)

        if self.kind == "int8":
            out = dict(A=raw(rows * k), B=raw(k * n).view(torch.int8),
                       D=torch.empty(rows * n, dtype=torch.int32, device=dev))
            out["C"] = (torch.randint(-1000, 1001, (rows * n,), dtype=torch.int32, device=dev, generator=g)
                        if self.beta != 0 else out["D"])
            if self.chain:
                out["bias"] = torch.randint(-(1 << 15), (1 << 15) + 1, (n,), dtype=torch.int32, device=dev,
                                            generator=g)
            return out
        per = 2 if self.fmt == _capi.FMT_E2M1 else 1
        kg = (k + 31) // 32

        def elements(r):
            x = raw(r * k // per)
            if self.fmt == _capi.FMT_E4M3:      # 0x7F / 0xFF are NaN
                x = torch.where((x & 0x7F) == 0x7F, x & 0xFE, x)
            elif self.fmt == _capi.FMT_E5M2:    # exponent 11111 is Inf / NaN
                x = torch.where((x & 0x7C) == 0x7C, x & 0xFB, x)
            return x

        def scales(r):
            return torch.randint(self.scale_lo, self.scale_hi + 1, (r * kg,), dtype=torch.uint8, device=dev,
                                 generator=g)

        out = dict(A=elements(rows), SA=scales(rows), B=elements(n), SB=scales(n),
                   D=torch.empty(rows * n, dtype=torch.float32, device=dev))
        out["C"] = (torch.randn(rows * n, dtype=torch.float32, device=dev, generator=g)
                    if self.beta != 0 else out["D"])
        return out

    def operator(self, **kw):
        import cpu_ops_b200 as c
        if self.kind == "int8":
            return c.GemmU8S8S32(c.RowMajor, c.RowMajor, c.RowMajor, **kw)
        st = {2: c.fp8e4m3_t, 3: c.fp8e5m2_t, 4: c.fp4e2m1_t}[self.fmt]
        return c.GemmMx(st, st, c.RowMajor, **kw)

    def arguments(self, op, bufs, rows=None):
        """bufs: dict name -> anything with a pointer (numpy array / torch tensor)."""
        import cpu_ops_b200 as c
        rows = self.m if rows is None else rows
        n, k = self.n, self.k
        if self.kind == "int8":
            chain = []
            if self.chain:
                chain = [c.BiasAdd(bufs["bias"]), c.Relu(), c.Clamp(0, 1 << 20)]
            epi = c.LinearCombinationFused(self.alpha, self.beta, chain)
            return op.Arguments(c.GemmCoord(rows, n, k), c.TensorRef(bufs["A"], k),
                                c.TensorRef(bufs["B"], n), c.TensorRef(bufs["C"], n),
                                c.TensorRef(bufs["D"], n), epi, self.split_k)
        kg = (k + 31) // 32
        return op.Arguments(c.GemmCoord(rows, n, k), c.MxTensorRef(bufs["A"], bufs["SA"], k, kg),
                            c.MxTensorRef(bufs["B"], bufs["SB"], k, kg), c.TensorRef(bufs["C"], n),
                            c.TensorRef(bufs["D"], n), c.LinearCombination(self.alpha, self.beta),
                            self.split_k)

    def reference_call(self, ref, h, rows, threads=0):
        """One call of the reference's CPU operator on host arrays `h`."""
        n, k = self.n, self.k
        if self.kind == "int8":
            if self.chain:
                return ref.gemm_u8s8s32_bias_relu_clamp(rows, n, k, h["A"], k, h["B"], n, h["C"], n,
                                                        h["D"], n, self.alpha, self.beta, h["bias"],
                                                        0, 1 << 20, self.split_k, threads)
            return ref.gemm_u8s8s32(rows, n, k, h["A"], k, True, h["B"], n, True, h["C"], n, h["D"],
                                    n, True, self.alpha, self.beta, False, self.split_k, threads)
        kg = (k + 31) // 32
        return ref.gemm_mx(rows, n, k, self.fmt, h["A"], h["SA"], k, kg, self.fmt, h["B"], h["SB"],
                           k, kg, h["C"], n, h["D"], n, True, self.alpha, self.beta, False,
                           self.split_k, threads)

    @property
    def dtype(self):
        from cpu_ops_b200 import _capi
        return {"int8": "u8*s8->s32"}.get(self.kind) or {
            _capi.FMT_E4M3: "mxfp8 e4m3 (f32 accumulate)", _capi.FMT_E5M2: "mxfp8 e5m2 (f32 accumulate)",
            _capi.FMT_E2M1: "mxfp4 e2m1 (f32 accumulate)"}[self.fmt]

    @property
    def peak_factor(self):
        """Dense tensor peak relative to bf16: int8/fp8 x2, fp4 x4."""
        from cpu_ops_b200 import _capi
        return 4.0 if (self.kind == "mx" and self.fmt == _capi.FMT_E2M1) else 2.0

    def roofline(self, seconds, peaks, peak_kind, rows=None):
        """Roofline of one launch that took `seconds`: the bound follows from the arithmetic
        intensity (ops per compulsory byte) against the machine balance of the measured
        peaks; the fraction is given against the measured and against the nominal peak."""
        ops, byts = self.ops(rows), self.min_bytes(rows)
        tensor_peak = self.peak_factor * float(peaks["bf16_tflops"])
        hbm_peak = float(peaks["hbm_gbs"])
        balance = tensor_peak * 1e12 / (hbm_peak * 1e9)
        bound = "hbm" if (self.bound == "hbm" or ops / byts < balance) else "tensor"
        if bound == "hbm":
            achieved = byts / seconds / 1e9 if seconds else None
            peak, nominal, unit = hbm_peak, NOMINAL_PEAKS["hbm_gbs"], "GB/s"
            basis = f"hbm_gbs ({peak_kind}); nominal 8000 GB/s"
        else:
            achieved = ops / seconds / 1e12 if seconds else None
            peak, nominal, unit = tensor_peak, NOMINAL_PEAKS[self.peak_factor], "TFLOP/s"
            sustained = self.peak_factor * float(peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]))
            basis = (f"{self.peak_factor:g} x bf16_tflops burst ({peak_kind}): dense "
                     f"{'fp4' if self.peak_factor == 4 else 'int8/fp8'} is nominally {self.peak_factor:g}x "
                     f"bf16 and no 8/4-bit peak was measured on this pool; nominal {nominal:g} TOP/s")
        out = {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit,
               "frac": (achieved / peak) if achieved else None,
               "peak_nominal": nominal, "frac_nominal": (achieved / nominal) if achieved else None}
        if bound == "tensor":
            # the same factor times the bf16 rate the GPU sustains under its power cap: the yardstick
            # for a kernel timed inside a long run of back-to-back calls
            out.update({"peak_sustained": sustained, "frac_sustained": (achieved / sustained) if achieved else None})
        out.update({
                "intensity_ops_per_byte": ops / byts, "balance_ops_per_byte": balance,
                "algorithmic_per_launch": byts if bound == "hbm" else ops, "peak_basis": basis})
        return out


# ---------------------------------------------------------------------------------
# CPU baseline: the reference's own operator on the host cores
# ---------------------------------------------------------------------------------
def time_reference(wl: Workload, steps: int, warmup: int, budget_s: float = 20.0):
    """Times oracle/_ref (the unmodified reference headers) the way the
    reference's benchmark does: warm-up, then wall clock around op(args) with
    all hardware threads (examples/01_benchmark.cc:25-35,96-101).  Each step is
    a bounded row-block sample of the workload."""
    from oracle.loader import Reference, have_reference
    if not have_reference():
        return None
    ref = Reference()
    # calibrate the sample so that the whole run stays near the budget
    rows = min(wl.m, 256)
    h = wl.host_operands(seed=1234, rows=rows)
    t0 = time.perf_counter()
    wl.reference_call(ref, h, rows)
    t_probe = max(time.perf_counter() - t0, 1e-4)
    per_row = t_probe / rows
    total_calls = max(1, steps + warmup)
    rows_budget = int(budget_s / total_calls / per_row)
    rows = max(min(wl.m, rows_budget), min(wl.m, 128))
    if rows >= 128:
        rows = rows // 128 * 128
    h = wl.host_operands(seed=1234, rows=rows)
    for _ in range(warmup):
        wl.reference_call(ref, h, rows)
    times = []
    t_all0 = time.perf_counter()
    for _ in range(steps):
        t0 = time.perf_counter()
        wl.reference_call(ref, h, rows)
        times.append(time.perf_counter() - t0)
    t_all = time.perf_counter() - t_all0
    return dict(rows=rows, mean_s=t_all / steps, best_s=min(times), isa=ref.isa,
                threads=ref.pool_threads, lib=ref.path.name)


def rate_of(wl: Workload, rows, seconds):
    if wl.bound == "hbm":
        return wl.min_bytes(rows) / seconds / 1e9, "GB/s"
    return wl.ops(rows) / seconds / 1e12, "TFLOP/s" if wl.kind == "mx" else "TOP/s"


# ---------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------
class ClockSampler(threading.Thread):
    """Samples SM clock and clock-event reasons of one GPU through NVML."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap", 0x80: "hw_power_brake", 0x2: "applications_clocks_setting"}

    def __init__(self, index, period_s=0.004):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.mark = [], None
        self._stop = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.max_mhz = None

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.samples.append((time.perf_counter(), mhz, reasons))
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._stop.set()

    def summary(self, t0, t1):
        inside = [s for s in self.samples if t0 <= s[0] <= t1] or self.samples
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        mhz = sorted(s[1] for s in inside)
        bits = 0
        for s in inside:
            bits |= s[2]
        reasons = [name for bit, name in self.REASONS.items() if bits & bit]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(inside)}


# ---------------------------------------------------------------------------------
def run_reference_arm(args, wl, rank, world):
    if rank != 0:
        return 0
    r = time_reference(wl, args.steps, args.warmup)
    if r is None:
        print(json.dumps({"impl": "reference",
                          "unavailable": "oracle/_ref is not built (reference checkout absent at build time)"}))
        return 0
    value, unit = rate_of(wl, r["rows"], r["mean_s"])
    sample = (f"{r['rows']} of {wl.m} output rows x N={wl.n} x K={wl.k} per step, "
              f"{r['lib']} ({r['isa']}), {r['threads']} threads")
    line = {
        "impl": "reference", "metric": metric_name(wl), "value": value, "unit": unit,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": r["mean_s"] * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
        "config": config_of(wl, world),
        "cpu_baseline": {"value": value, "unit": unit, "cores": r["threads"], "kind": "reference",
                         "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))
    return 0


def metric_name(wl):
    if wl.bound == "hbm":
        return f"decode GEMM HBM GB/s ({wl.name})"
    return f"{'int8' if wl.kind == 'int8' else ('mxfp4' if wl.peak_factor == 4 else 'mxfp8')} GEMM " \
           f"{'TOPS' if wl.kind == 'int8' else 'TFLOPS'} ({wl.name}, whole job)"


def config_of(wl, world):
    return {"workload": wl.name, "m_per_gpu": wl.m, "n": wl.n, "k": wl.k, "alpha": wl.alpha,
            "beta": wl.beta, "layout": "TN" if wl.kind == "mx" else "all RowMajor",
            "sharding": f"output row blocks over {world} rank(s), B replicated, no collective",
            "l2": "operands rotate over distinct buffer sets (at least 3) whose total size exceeds "
                  "twice the L2"}


TABLE_WORKLOADS = ("int8_2048", "mxfp8_e4m3_4096", "mxfp4_decode_m1", "mxfp4_decode_m8", "mxfp4_decode_m32",
                   "int8_8192_chain", "mx_e5m2_16384", "mx_e2m1_16384", "int8_8192", "mxfp8_8192", "mxfp4_8192")


def run_table(args):
    """One line per workload, in the manner of the reference's benchmark program
    (examples/01_benchmark.cc:204-343 prints name, shape, best time and rate per config):
    device-resident operands over rotating sets larger than the L2, best and median of `--steps` calls
    timed one by one with CUDA events.  A survey, not the contract line."""
    import torch
    import cpu_ops_b200 as c
    from cpu_ops_b200 import _capi
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks, _ = load_peaks()
    stream = torch.cuda.current_stream().cuda_stream
    print(f"{'workload':18s} {'m':>6s} {'n':>6s} {'k':>6s} {'plan':>14s} {'best us':>10s} {'median us':>10s} "
          f"{'rate (best)':>16s} {'of peak':>8s}")
    for name in TABLE_WORKLOADS:
        wl = Workload(name)
        host = wl.host_operands(seed=0)
        set_bytes = sum(v.nbytes for v in host.values())
        l2_bytes = torch.cuda.get_device_properties(dev).L2_cache_size
        n_sets = max(2, -(-2 * l2_bytes // set_bytes) + 1)  # one trip round the ring outgrows the L2
        sets = [{k_: torch.from_numpy(v).to(dev)
                 for k_, v in (host if s_ == 0 else wl.host_operands(seed=s_)).items()} for s_ in range(n_sets)]
        op = wl.operator(stream=stream, asynchronous=True, memory_space=_capi.MEM_DEVICE)
        descs = [op.describe(wl.arguments(op, b)) for b in sets]
        for i in range(max(4, n_sets)):
            assert op.run(descs[i % n_sets]) == c.Status.kSuccess, _capi.last_error()
        torch.cuda.synchronize()
        times = []
        for i in range(max(5, args.steps)):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            op.run(descs[i % n_sets])
            e1.record()
            e1.synchronize()
            times.append(e0.elapsed_time(e1) * 1e-3)
        times.sort()
        best, med = times[0], times[len(times) // 2]
        rate, unit = rate_of(wl, wl.m, best)
        peak = float(peaks["hbm_gbs"]) if wl.bound == "hbm" else wl.peak_factor * float(peaks["bf16_tflops"])
        plan = _capi.last_plan()
        tile = f"{256 if plan.pair else 128}x{plan.tile_n}" + (f"/k{plan.slices}" if plan.slices > 1 else "")
        print(f"{name:18s} {wl.m:6d} {wl.n:6d} {wl.k:6d} {tile:>14s} {best * 1e6:10.1f} {med * 1e6:10.1f} "
              f"{rate:10.1f} {unit:>5s} {rate / peak:8.2f}")
        del sets, descs
        torch.cuda.empty_cache()
    return 0


def plan_dict(plan, graph=False):
    return {"tile": f"{256 if plan.pair else 128}x{plan.tile_n}", "cta_pair": bool(plan.pair),
            "operands_swapped": bool(plan.swapped), "k_slices": plan.slices, "smem_stages": plan.stages,
            "ctas": plan.grid, "prepared_b": bool(plan.prepared_b), "small_m_kernel": bool(plan.decode),
            "cuda_graph": bool(graph)}


def _event_ms(fn, count):
    import torch
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(count):
        fn(i)
    e1.record()
    e1.synchronize()
    return e0.elapsed_time(e1) / count


def measure_workload(wl, dev, lib, peaks, peak_kind, budget_s=0.1, with_graph=False, sampler=None):
    """One suite record: device-resident operands generated on the device, rotating over
    enough distinct sets that one trip touches more than twice the L2; the call time back to
    back (mean of three passes; the best pass is reported beside it), the dominant kernel's
    own time (CUDA events around it), and for the decode shapes the same calls replayed from
    a CUDA graph."""
    import ctypes as C
    import torch
    import cpu_ops_b200 as c
    from cpu_ops_b200 import _capi
    l2_bytes = torch.cuda.get_device_properties(dev).L2_cache_size
    first = wl.device_operands(dev, seed=17)
    set_bytes = sum(v.numel() * v.element_size() for k_, v in first.items() if k_ != "C" or v is not first["D"])
    n_sets = max(2, -(-2 * l2_bytes // set_bytes) + 1)
    sets = [first] + [wl.device_operands(dev, seed=17 + i) for i in range(1, n_sets)]
    stream = torch.cuda.current_stream().cuda_stream
    op = wl.operator(stream=stream, asynchronous=True, memory_space=_capi.MEM_DEVICE)
    descs = [op.describe(wl.arguments(op, b)) for b in sets]

    def call(i):
        st = op.run(descs[i % n_sets])
        if st != c.Status.kSuccess:
            raise RuntimeError(f"{wl.name}: GEMM failed: {st!r}: {_capi.last_error()}")

    launches0 = c.launch_count()
    for i in range(max(3, n_sets)):
        call(i)
    torch.cuda.synchronize()
    launches_per_call = (c.launch_count() - launches0) / max(3, n_sets)
    if c.stream_status(stream) != c.Status.kSuccess:
        raise RuntimeError(f"{wl.name}: device-side error: {_capi.last_error()}")
    plan = _capi.last_plan()
    est_ms = _event_ms(call, 3)
    steps = int(min(2000, max(10, budget_s * 1e3 / max(est_ms, 1e-3))))
    t_pass0 = time.perf_counter()
    passes = [_event_ms(call, steps)]
    # the dominant kernel alone, between the passes (same thermal / power state): CUDA events
    # around every launch of it, which for a kernel of a few microseconds also bracket the
    # launch gap the events themselves open (no overlap with its neighbours)
    lib.cpuops_b200_profile(1)
    for i in range(min(steps, 100)):
        call(i)
    torch.cuda.synchronize()
    lib.cpuops_b200_profile(0)
    kms, kn = C.c_double(0), C.c_int32(0)
    lib.cpuops_b200_profile_collect(C.byref(kms), C.byref(kn))
    kernel_ms = kms.value / kn.value if kn.value else None
    passes += [_event_ms(call, steps) for _ in range(2)]
    clk = sampler.summary(t_pass0, time.perf_counter()) if sampler is not None else None
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(min(steps, 32)):   # few enough that the launch queue never pushes back
        call(i)
    host_us = (time.perf_counter() - t0) / min(steps, 32) * 1e6   # issue cost on the host
    torch.cuda.synchronize()
    mean_ms, best_ms = sum(passes) / len(passes), min(passes)
    rate, unit = rate_of(wl, wl.m, mean_ms / 1e3)
    rec = {"workload": wl.name, "m": wl.m, "n": wl.n, "k": wl.k, "alpha": wl.alpha, "beta": wl.beta,
           "dtype": wl.dtype, "operand_sets": n_sets, "steps_per_pass": steps,
           "ms_per_call": mean_ms, "ms_per_call_best_pass": best_ms, "ms_per_call_passes": passes,
           "host_issue_us_per_call": host_us, "launches_per_call": launches_per_call,
           "kernel_ms": kernel_ms,
           "kernel_ms_how": "CUDA events around each launch of the dominant kernel (for kernels of a few "
                            "microseconds this includes the launch gap that the events open)",
           "value": rate, "unit": unit, "kernel_plan": plan_dict(plan), "clocks": clk,
           "roofline": wl.roofline(mean_ms / 1e3, peaks, peak_kind),
           "roofline_kernel": wl.roofline(kernel_ms / 1e3, peaks, peak_kind) if kernel_ms else None}
    if with_graph:
        # The same calls replayed from a CUDA graph: what a launch-bound decode loop would do.
        # The capture stream runs the calls once before the capture begins (workspace, counters).
        side = torch.cuda.Stream(device=dev)
        op_g = wl.operator(stream=side.cuda_stream, asynchronous=True, memory_space=_capi.MEM_DEVICE)
        descs_g = [op_g.describe(wl.arguments(op_g, b)) for b in sets]
        with torch.cuda.stream(side):
            for dsc in descs_g:
                op_g.run(dsc)
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side, capture_error_mode="relaxed"):
                for dsc in descs_g:
                    st = op_g.run(dsc)
                    if st != c.Status.kSuccess:
                        raise RuntimeError(f"{wl.name}: capture failed: {st!r}: {_capi.last_error()}")
            for _ in range(3):
                graph.replay()
            side.synchronize()
            trips = max(3, steps // n_sets)
            best_g = min(_event_ms(lambda i: graph.replay(), trips) for _ in range(3)) / n_sets
        rec["graph_ms_per_call"] = best_g
        rec["roofline_graph"] = wl.roofline(best_g / 1e3, peaks, peak_kind)
        del graph
    del sets, descs
    torch.cuda.empty_cache()
    return rec


def run_suite(dev, lib, peaks, peak_kind, device_index=0):
    out = []
    sampler = ClockSampler(device_index)
    sampler.start()
    for name in TABLE_WORKLOADS:
        wl = Workload(name)
        out.append(measure_workload(wl, dev, lib, peaks, peak_kind, with_graph=wl.bound == "hbm", sampler=sampler))
    sampler.stop()
    return out


# ---------------------------------------------------------------------------------
# N > 1: the 16384^3 MX problems, output row blocks over the ranks
# ---------------------------------------------------------------------------------
def _decode_f64(fmt, codes):
    """Exact decode of MX element codes to float64 (numpy): e5m2 is the upper byte of an
    IEEE half, e4m3 / e2m1 by table."""
    from cpu_ops_b200 import _capi
    codes = np.asarray(codes, dtype=np.uint8)
    if fmt == _capi.FMT_E5M2:
        return (codes.astype(np.uint16) << 8).view(np.float16).astype(np.float64)
    if fmt == _capi.FMT_E2M1:
        mag = np.array([0, .5, 1, 1.5, 2, 3, 4, 6], np.float64)
        return np.where(codes & 8, -1.0, 1.0) * mag[codes & 7]
    e, mnt = (codes >> 3) & 0xF, (codes & 7).astype(np.float64)
    val = np.where(e == 0, mnt * 2.0 ** -9, (8 + mnt) * 2.0 ** (e.astype(np.float64) - 10))
    return np.where(codes & 0x80, -val, val)


def sampled_f64_reference(wl, A_rows, SA_rows, B_rows, SB_rows):
    """D[i, j] in double for the given operand rows (host arrays: elements as stored, scales
    one byte per 32 k): decode exactly, apply the E8M0 scales, accumulate in float64 -- the
    arithmetic of the reference's own test (test/test_gemm_mx.cc:181-197), written here in
    numpy so that the bench needs nothing from the test-side oracle."""
    from cpu_ops_b200 import _capi
    k = wl.k

    def expand(data, scl):
        r = data.shape[0]
        if wl.fmt == _capi.FMT_E2M1:
            lo, hi = data & 0xF, data >> 4
            codes = np.stack([lo, hi], axis=-1).reshape(r, k)   # even k in the low nibble
        else:
            codes = data.reshape(r, k)
        sc = np.exp2(scl.reshape(r, k // 32).astype(np.float64) - 127.0)
        return _decode_f64(wl.fmt, codes) * np.repeat(sc, 32, axis=1)

    return wl.alpha * (expand(A_rows, SA_rows) @ expand(B_rows, SB_rows).T)


def run_sharded(args, rank, world, dev, lib, peaks, peak_kind):
    """Each 16384^3 MX problem cut into output row blocks (cpuops_b200_shard_rows); every rank
    holds its rows of A and all of B.  Timed: the GEMM steps alone, and the same steps each
    followed by an all-gather of the D blocks into a replicated D (NCCL, on a second stream,
    two D buffers, so the gather of step i runs under the GEMM of step i + 1).  Checked,
    outside the timed region: sampled elements of every rank's block against a float64
    reference on the CPU, and the first rows of every block, bit for bit, against rank 0's
    single-GPU computation of the same rows."""
    import torch
    import torch.distributed as dist
    import cpu_ops_b200 as c
    from cpu_ops_b200 import _capi, sharding
    out = {}
    steps = max(5, min(args.steps, 20))
    for name in ("mx_e5m2_16384", "mx_e2m1_16384"):
        wl = Workload(name)
        M, n, k = wl.m, wl.n, wl.k
        per = 2 if wl.fmt == _capi.FMT_E2M1 else 1
        kg = k // 32
        sh = sharding.shard_rows(M, world, rank)
        r0, rn = sh.row_begin, sh.row_count
        assert rn * world == M, "the bench assumes equal row blocks"
        full = wl.device_operands(dev, seed=0xC5C5 + wl.fmt)   # the whole problem, identical on every rank
        a_rows = lambda lo, cnt: full["A"][lo * k // per:(lo + cnt) * k // per]
        sa_rows = lambda lo, cnt: full["SA"][lo * kg:(lo + cnt) * kg]
        d_blk = [torch.empty(rn * n, dtype=torch.float32, device=dev) for _ in range(2)]
        stream = torch.cuda.current_stream().cuda_stream
        op = wl.operator(stream=stream, asynchronous=True, memory_space=_capi.MEM_DEVICE)

        def describe(lo, cnt, dbuf):
            bufs = dict(A=a_rows(lo, cnt), SA=sa_rows(lo, cnt), B=full["B"], SB=full["SB"], C=dbuf, D=dbuf)
            return op.describe(wl.arguments(op, bufs, rows=cnt))

        descs = [describe(r0, rn, d_blk[j]) for j in range(2)]

        def gemm(i):
            st = op.run(descs[i % 2])
            if st != c.Status.kSuccess:
                raise RuntimeError(f"sharded {name}: GEMM failed: {st!r}: {_capi.last_error()}")

        def timed(fn, count):
            dist.barrier()
            torch.cuda.synchronize()
            ms = _event_ms(fn, count)
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())

        for i in range(3):
            gemm(i)
        gemm_ms = timed(gemm, steps)
        plan = _capi.last_plan()

        # with the all-gather of D: gather of step i on a second stream under GEMM i + 1
        d_full = [torch.empty(M * n, dtype=torch.float32, device=dev) for _ in range(2)]
        side = torch.cuda.Stream(device=dev)
        ready = [torch.cuda.Event() for _ in range(2)]
        done = [None, None]

        def gemm_then_gather(i):
            j = i % 2
            if done[j] is not None:
                torch.cuda.current_stream().wait_event(done[j])   # the gather that read d_blk[j] is over
            gemm(i)
            ready[j].record(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                side.wait_event(ready[j])
                dist.all_gather_into_tensor(d_full[j], d_blk[j])
                if done[j] is None:
                    done[j] = torch.cuda.Event()
                done[j].record(side)

        def gathered(count):
            def body(i):
                gemm_then_gather(i)
                if i == count - 1:
                    torch.cuda.current_stream().wait_stream(side)
            return body

        for i in range(3):
            gemm_then_gather(i)
        torch.cuda.current_stream().wait_stream(side)
        with_gather_ms = timed(gathered(steps), steps)
        # the same with 32 SMs left to the gather: the GEMM's persistent CTAs otherwise hold
        # every SM until the kernel ends, and NCCL's kernel can only start after it
        sm_total = torch.cuda.get_device_properties(dev).multi_processor_count
        lib.cpuops_b200_set_sm_limit(-1, sm_total - 32)
        for i in range(3):
            gemm_then_gather(i)
        torch.cuda.current_stream().wait_stream(side)
        with_gather_margin_ms = timed(gathered(steps), steps)
        gemm_margin_ms = timed(gemm, steps)
        lib.cpuops_b200_set_sm_limit(-1, 0)
        gather_ms = timed(lambda i: dist.all_gather_into_tensor(d_full[0], d_blk[0]), steps)

        # ---- checks (not timed) ----
        torch.cuda.synchronize()
        gemm(0)
        torch.cuda.synchronize()
        D = d_blk[0].view(rn, n)
        # the replicated D really is the blocks in rank order
        dist.all_gather_into_tensor(d_full[0], d_blk[0])
        torch.cuda.synchronize()
        gather_ok = bool(torch.equal(d_full[0].view(M, n)[r0:r0 + rn].view(torch.int32), D.view(torch.int32)))
        # (1) sampled positions against float64 on the CPU
        gsel = torch.Generator(device="cpu")
        gsel.manual_seed(1234 + rank)
        ri = torch.randperm(rn, generator=gsel)[:16].sort().values
        cj = torch.randperm(n, generator=gsel)[:64].sort().values
        A_h = full["A"].view(M, k // per)[r0 + ri.to(dev)].cpu().numpy()
        SA_h = full["SA"].view(M, kg)[r0 + ri.to(dev)].cpu().numpy()
        B_h = full["B"].view(n, k // per)[cj.to(dev)].cpu().numpy()
        SB_h = full["SB"].view(n, kg)[cj.to(dev)].cpu().numpy()
        want = sampled_f64_reference(wl, A_h, SA_h, B_h, SB_h)
        got = D[ri.to(dev)][:, cj.to(dev)].cpu().numpy().astype(np.float64)
        err = float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-300))
        # (2) the first rows of every block, bit for bit, against rank 0 computing them alone
        sub = min(1024, rn)
        mine = D[:sub].contiguous().view(-1)
        everyone = torch.empty(world * sub * n, dtype=torch.float32, device=dev)
        dist.all_gather_into_tensor(everyone, mine)
        bits_ok = True
        if rank == 0:
            alone = torch.empty(sub * n, dtype=torch.float32, device=dev)
            for j in range(world):
                rj = sharding.shard_rows(M, world, j).row_begin
                st = op.run(describe(rj, sub, alone))
                torch.cuda.synchronize()
                bits_ok = bits_ok and st == c.Status.kSuccess and bool(
                    torch.equal(alone.view(torch.int32), everyone[j * sub * n:(j + 1) * sub * n].view(torch.int32)))
        flags = torch.tensor([1.0 if (err <= 1e-5 and bits_ok and gather_ok) else 0.0, -err], device=dev,
                             dtype=torch.float64)
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
        # the whole problem on one GPU, for the strong-scaling ratio (rank 0 only; others wait)
        single_ms = None
        if rank == 0:
            d_whole = d_full[1]
            whole = describe(0, M, d_whole)
            for _ in range(2):
                op.run(whole)
            torch.cuda.synchronize()
            single_ms = _event_ms(lambda i: op.run(whole), 5)
        dist.barrier()
        if c.stream_status(stream) != c.Status.kSuccess:
            raise RuntimeError(f"sharded {name}: device-side error: {_capi.last_error()}")
        if rank == 0:
            ops = wl.ops()
            blk_bytes = rn * n * 4
            out[name] = {
                "m": M, "n": n, "k": k, "rows_per_rank": rn, "steps": steps, "kernel_plan": plan_dict(plan),
                "ms_per_step": gemm_ms, "tflops_aggregate": ops / (gemm_ms / 1e3) / 1e12,
                "tflops_per_gpu": ops / world / (gemm_ms / 1e3) / 1e12,
                "single_gpu_ms_per_step": single_ms,
                "strong_scaling_efficiency": single_ms / (world * gemm_ms),
                "with_gather": {"ms_per_step": with_gather_ms,
                                "tflops_aggregate": ops / (with_gather_ms / 1e3) / 1e12,
                                "strong_scaling_efficiency": single_ms / (world * with_gather_ms)},
                "with_gather_32_sms_left_to_nccl": {
                    "ms_per_step": with_gather_margin_ms, "gemm_alone_ms_per_step": gemm_margin_ms,
                    "tflops_aggregate": ops / (with_gather_margin_ms / 1e3) / 1e12,
                    "strong_scaling_efficiency": single_ms / (world * with_gather_margin_ms),
                    "how": "cpuops_b200_set_sm_limit(SMs - 32): the GEMM leaves 32 SMs free (NCCL's "
                           "all-gather kernel is 32 CTAs wide here), so the gather of step i runs beside "
                           "the GEMM of step i + 1"},
                "gather_alone": {"ms": gather_ms, "bytes_received_per_rank": (world - 1) * blk_bytes,
                                 "nvlink_gbs_received_per_rank": (world - 1) * blk_bytes / (gather_ms / 1e3) / 1e9},
                "parity_ok": bool(flags[0].item() == 1.0), "worst_sampled_normwise_error": float(-flags[1].item()),
                "parity_checks": "per rank: 16 x 64 sampled elements vs a float64 CPU reference (<= 1e-5 "
                                 "normwise); first 1024 rows of every block bit-identical to rank 0's "
                                 "single-GPU run of those rows; gathered D equals the blocks in rank order",
                "l2": "per-rank inputs (A rows + all of B) exceed the L2",
            }
        del full, d_blk, d_full
        torch.cuda.empty_cache()
    return out



def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="mxfp8_e4m3_4096")
    ap.add_argument("--tile-n", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--table", action="store_true",
                    help="survey of every workload on one GPU (best / median call time), instead of the "
                         "JSON contract line")
    ap.add_argument("--gather", action="store_true",
                    help="N > 1: every step also all-gathers the ranks' D row blocks into a replicated D "
                         "(NCCL, on a second stream so that it overlaps the next step's GEMM)")
    ap.add_argument("--graph", action="store_true",
                    help="replay the calls from a CUDA graph (one trip round the operand ring per "
                         "replay), as a launch-bound decode loop would; steps are rounded to whole trips")
    ap.add_argument("--no-suite", action="store_true",
                    help="N = 1: skip the per-workload `suite` records (headline only)")
    ap.add_argument("--no-sharded", action="store_true",
                    help="N > 1: skip the row-sharded 16384^3 `sharded` leg (headline only)")
    ap.add_argument("--prepared-b", action="store_true",
                    help="MX workloads: register each B operand once (cpuops_b200_prepare_b), as a "
                         "decode loop with fixed weights would")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    wl = Workload(args.workload)

    if args.impl == "reference":
        return run_reference_arm(args, wl, rank, world)
    if args.table:
        return run_table(args)

    import torch
    import torch.distributed as dist
    import cpu_ops_b200 as c
    from cpu_ops_b200 import _capi

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback in the product)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    lib = _capi.load()
    peaks, peak_kind = load_peaks()

    # ---- operands: rotating device sets (distinct data), this rank's row block ----
    # At least three sets, and enough of them that one trip round the ring touches
    # more than twice the L2's capacity, so no launch finds its operands cached.
    host0 = wl.host_operands(seed=1000 * rank)
    set_bytes = sum(v.nbytes for v in host0.values())
    l2_bytes = torch.cuda.get_device_properties(dev).L2_cache_size
    n_sets = max(3, -(-2 * l2_bytes // set_bytes) + 1)
    sets = []
    for s in range(n_sets):
        h = host0 if s == 0 else wl.host_operands(seed=1000 * rank + s)
        sets.append({k_: torch.from_numpy(v).to(dev) for k_, v in h.items()})
    stream = torch.cuda.current_stream().cuda_stream
    op = wl.operator(stream=stream, asynchronous=True, tile_n=args.tile_n,
                     memory_space=_capi.MEM_DEVICE)
    # descriptors are built once, as a C++ caller's Arguments would be; a step is one call
    descs = [op.describe(wl.arguments(op, b)) for b in sets]
    prepared = []
    if args.prepared_b and wl.kind == "mx":
        prepared = [c.PreparedB(op, wl.arguments(op, b)) for b in sets]

    gather_stream, gather_events, gather_done, d_full = None, [], [], None
    if args.gather and world > 1:
        # equal blocks (every rank holds wl.m rows): in-place all-gather into a full-size D
        gather_stream = torch.cuda.Stream(device=dev)
        gather_events = [torch.cuda.Event() for _ in range(n_sets)]
        gather_done = [None] * n_sets  # set j's D may be overwritten once its gather has read it
        d_full = [torch.empty((world * wl.m * wl.n,), dtype=sets[0]["D"].dtype, device=dev)
                  for _ in range(2)]

    def direct_step(i):
        j = i % n_sets
        if gather_stream is not None and gather_done[j] is not None:
            torch.cuda.current_stream().wait_event(gather_done[j])
        st = op.run(descs[j])
        if st != c.Status.kSuccess:
            raise RuntimeError(f"GEMM failed: {st!r}: {_capi.last_error()}")
        if gather_stream is not None:
            gather_events[j].record(torch.cuda.current_stream())
            with torch.cuda.stream(gather_stream):
                gather_stream.wait_event(gather_events[j])
                dist.all_gather_into_tensor(d_full[i % 2], sets[j]["D"])
                if gather_done[j] is None:
                    gather_done[j] = torch.cuda.Event()
                gather_done[j].record(gather_stream)

    step = direct_step
    graph, launches_per_trip = None, 0
    if args.graph:
        # Capture one call per operand set.  The capture stream first runs every call once
        # outside capture: the library's calls are plain kernel launches once its workspace
        # for that stream exists, and it refuses to allocate while a capture is under way.
        args.steps = max(n_sets, args.steps // n_sets * n_sets)
        args.warmup = max(n_sets, args.warmup // n_sets * n_sets)
        cap = torch.cuda.Stream(device=dev)
        op_g = wl.operator(stream=cap.cuda_stream, asynchronous=True, tile_n=args.tile_n,
                           memory_space=_capi.MEM_DEVICE)
        descs_g = [op_g.describe(wl.arguments(op_g, b)) for b in sets]
        with torch.cuda.stream(cap):
            for dsc in descs_g:
                op_g.run(dsc)
            cap.synchronize()
        graph = torch.cuda.CUDAGraph()
        launches_before_capture = c.launch_count()
        with torch.cuda.graph(graph, stream=cap, capture_error_mode="relaxed"):
            for dsc in descs_g:
                st = op_g.run(dsc)
                if st != c.Status.kSuccess:
                    raise RuntimeError(f"GEMM failed during capture: {st!r}: {_capi.last_error()}")

        launches_per_trip = c.launch_count() - launches_before_capture

        def step(i):  # one replay covers n_sets steps
            if i % n_sets == 0:
                graph.replay()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    sampler.start()
    for i in range(args.warmup):
        step(i)
    barrier()
    if c.stream_status(stream) != c.Status.kSuccess:
        raise RuntimeError("device-side error during warm-up: " + _capi.last_error())
    plan = _capi.last_plan()
    launches0 = c.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall0 = time.perf_counter()
    ev0.record()
    for i in range(args.steps):
        step(i)
    if gather_stream is not None:
        torch.cuda.current_stream().wait_stream(gather_stream)
    ev1.record()
    barrier()
    launches = c.launch_count() - launches0
    if graph is not None:  # replayed launches do not pass through the library's counter
        launches = launches_per_trip * (args.steps // n_sets)
    ms = ev0.elapsed_time(ev1)
    # The same K steps again, directly after the timed region, with the library's
    # per-launch events around the tensor-core kernel (on the launching stream): the
    # roofline's duration.  Kept out of the timed region because an event between the
    # scale re-layout and the GEMM launch would serialise the two kernels.
    import ctypes as C
    lib.cpuops_b200_profile(1)
    for i in range(args.steps):
        direct_step(i)
    barrier()
    t_wall1 = time.perf_counter()
    lib.cpuops_b200_profile(0)
    kms, kn = C.c_double(0), C.c_int32(0)
    lib.cpuops_b200_profile_collect(C.byref(kms), C.byref(kn))
    if c.stream_status(stream) != c.Status.kSuccess:
        raise RuntimeError("device-side error during the timed region: " + _capi.last_error())
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    clocks = sampler.summary(t_wall0, t_wall1)

    # ---- end to end: pinned host buffers through the synchronous call ----
    e2e = None
    if not args.no_e2e:
        pinned = {k_: torch.from_numpy(v).pin_memory() for k_, v in host0.items()}
        op_sync = wl.operator(tile_n=args.tile_n)
        a_sync = wl.arguments(op_sync, pinned)
        e2e_steps = max(3, min(args.steps, 30))
        for _ in range(2):
            op_sync(a_sync)
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            st = op_sync(a_sync)
            if st != c.Status.kSuccess:
                raise RuntimeError(f"e2e GEMM failed: {st!r}: {_capi.last_error()}")
        t_e2e = time.perf_counter() - t0
        if world > 1:
            t = torch.tensor([t_e2e], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            t_e2e = float(t.item())
        h2d = sum(v.numel() * v.element_size() for k_, v in pinned.items()
                  if k_ != "D" and not (k_ == "C" and wl.beta == 0))
        d2h = pinned["D"].numel() * pinned["D"].element_size()
        ev, eu = rate_of(wl, wl.m * world, t_e2e / e2e_steps)
        e2e = {"value": ev, "unit": eu, "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
               "ms_per_step": t_e2e / e2e_steps * 1e3, "steps": e2e_steps}
    sampler.stop()

    # ---- the other workloads (N = 1) / the row-sharded 16384^3 problems (N > 1) ----
    del sets, descs
    torch.cuda.empty_cache()
    suite = sharded = None
    if world == 1 and not args.no_suite and not args.graph:
        suite = run_suite(dev, lib, peaks, peak_kind, local_rank)
    if world > 1 and not args.no_sharded:
        sharded = run_sharded(args, rank, world, dev, lib, peaks, peak_kind)

    if rank == 0:
        sec_per_step = ms / 1e3 / args.steps
        value, unit = rate_of(wl, wl.m * world, sec_per_step)
        # roofline of the dominant (tensor-core) kernel, per launch
        k_avg_s = (kms.value / 1e3 / kn.value) if kn.value else None
        roofline = wl.roofline(k_avg_s, peaks, peak_kind)
        plan_now = plan_dict(plan, args.graph)
        cap = KERNEL_DRAM_TRAFFIC.get(wl.name)
        traffic_ok = cap is not None and cap["tile"] == plan_now["tile"] and cap["k_slices"] == plan_now["k_slices"]
        roofline.update({
            "traffic": cap["bytes"] if traffic_ok else None,
            "traffic_source": (f"ncu capture summarised in {cap['capture']} (dram__bytes_read.sum + "
                               f"dram__bytes_write.sum per launch, plan {cap['tile']})" if traffic_ok else
                               "no ncu capture of this kernel plan is on file"),
            "kernel": "decode_mx_kernel" if plan.decode else "gemm_tcgen05_kernel",
            "kernel_ms": (k_avg_s * 1e3) if k_avg_s else None, "timed_launches": kn.value,
            "timed_in": "the K steps repeated directly after the timed region, CUDA events "
                        "around each launch of this kernel on the launching stream"})
        line = {
            "metric": metric_name(wl), "value": value, "unit": unit, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype,
            "data": "synthetic",
            "config": dict(config_of(wl, world), kernel_plan=plan_now,
                gather_d=bool(args.gather and world > 1),
                seeds=f"operand set s of rank r: 1000*r + s (numpy PCG64 streams per operand, "
                      f"cpu_ops_b200/workloads.py)"),
            "clocks": clocks,
            "gpu_launches": int(launches), "roofline": roofline, "impl": "b200",
        }
        if e2e:
            line["e2e"] = e2e
        if suite is not None:
            line["suite"] = suite
        if sharded is not None:
            line["sharded"] = sharded
        if world == 1 and not args.no_cpu_baseline:
            r = time_reference(wl, steps=3, warmup=1, budget_s=15.0)
            if r is not None:
                cv, cu = rate_of(wl, r["rows"], r["best_s"])
                line["cpu_baseline"] = {
                    "value": cv, "unit": cu, "cores": r["threads"], "kind": "reference",
                    "sample": f"{r['rows']} of {wl.m} output rows x N={wl.n} x K={wl.k}, best of 3, "
                              f"{r['lib']} ({r['isa']})"}
            else:
                line["cpu_baseline"] = {"value": None, "unit": unit, "cores": 0, "kind": "reference",
                                        "sample": "oracle/_ref not built"}
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu
# captures summarised under profiles/, with the launch plan each capture was taken under: the
# figure is only quoted for a run that launches the same plan.
KERNEL_DRAM_TRAFFIC = {
    "mxfp8_e4m3_4096": {"bytes": 106.32e6 + 37.62e6, "tile": "256x224", "k_slices": 1,
                        "capture": "profiles/gemm_tcgen05_kernel_mxfp8_e4m3_4096.md"},
    "int8_8192": {"bytes": 306.31e6 + 239.16e6, "tile": "256x256", "k_slices": 1,
                  "capture": "profiles/gemm_tcgen05_kernel_int8_8192.md"},
    "int8_2048": {"bytes": 25.24e6, "tile": "128x256", "k_slices": 1,
                  "capture": "profiles/gemm_tcgen05_kernel_int8_2048.md"},
    "mxfp4_decode_m8": {"bytes": 31.30e6, "tile": "128x32", "k_slices": 1,
                        "capture": "profiles/decode_mx_kernel_mxfp4_decode_m8.md"},
}

if __name__ == "__main__":
    sys.exit(main())
