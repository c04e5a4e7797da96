#!/usr/bin/env python
"""Benchmark of the fused SwiGLU MLP forward on B200: `python bench.py --gpus N --steps K --warmup W`.

One "step" is one forward pass out = (silu(x Wg^T) * (x Wu^T)) Wd^T over one batch of synthetic
bf16 input (x ~ N(0,1), weights ~ N(0, 0.02^2), seeded, generated on the device).

  every N   workload c4: Llama-3-70B MLP prefill, M=8192, d=8192, F=28672.  N = 1: one GPU runs it whole.
            N > 1: Megatron tensor-parallel over the N ranks (W_gate/W_up column-split, W_down row-split,
            reduction of the output over NVLink); total work is fixed as N grows ("scaling": "strong").
            Launch N > 1 with torchrun, one rank per GPU.
  --workload  c2 (7B prefill), c3 (8B small-batch, M = 1/4/16/64, HBM roofline), c5 (ragged 13B shape,
            M = 32414 with x50 outliers) select the other benchmark configurations; at N = 1 the default
            run also measures c2 and c3 and reports them as sub-records ("also").

The JSON line printed by rank 0 carries
  value     whole-job TFLOP/s (6*M*d*F flops per step) with inputs resident in HBM, timed with CUDA
            events on the launching stream over exactly K steps, max over ranks;
  e2e       the same metric through the host-buffer entry point: every step copies x from pinned host
            memory to the device and the result back, inside the timed region;
  roofline  of the dominant kernel (the gate-up tcgen05 GEMM, two thirds of the flops): algorithmic
            flops per launch / its mean launch duration (CUDA events around each launch inside the timed
            region) against the measured dense-bf16 peak in MEASURED_PEAKS.json;
  parity    rows of the last timed step's output against the CPU oracle (fp32 expression), and for
            N > 1 whether every rank holds identical bits;
  sustained a second timed region of at least two seconds (clock-limited regime) with the SM clock sampled;
  gpu_baselines  (N = 1) torch bf16 eager on the same GPU, and the reference project's own kernel rebuilt
            for sm_100a on its own benchmark problem, next to this library's kernel on that problem;
  cpu_baseline  (N = 1) the eager PyTorch expression in fp32 on this box's host cores, on a row slab.

`--impl reference` times only that CPU expression (the reference project's own oracle arithmetic is its
only CPU path; its CUDA kernel covers the gate-up half only) and prints the same line shape.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "fused-swiglu_b200"))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "fused SwiGLU MLP fwd TFLOP/s"
UNIT = "TFLOP/s"
RAGGED_M = 32414  # sum of 32 lengths uniform in [1, 2048], torch.Generator().manual_seed(0)
WORKLOADS = {
    "c2_llama2_7b_prefill": dict(M=4096, d=4096, F=11008),
    "c4_llama3_70b_prefill": dict(M=8192, d=8192, F=28672),
    "c5_ragged_13b": dict(M=RAGGED_M, d=5120, F=13824),
    # small-batch (HBM-bound) configurations: single GPU only, roofline = HBM bandwidth
    "c3_llama3_8b_decode_m1": dict(M=1, d=4096, F=14336),
    "c3_llama3_8b_decode_m4": dict(M=4, d=4096, F=14336),
    "c3_llama3_8b_decode_m16": dict(M=16, d=4096, F=14336),
    "c3_llama3_8b_decode_m64": dict(M=64, d=4096, F=14336),
}
DEFAULT_WORKLOAD = "c4_llama3_70b_prefill"
ALSO_AT_ONE_GPU = ["c2_llama2_7b_prefill", "c3_llama3_8b_decode_m1", "c3_llama3_8b_decode_m16",
                   "c3_llama3_8b_decode_m64"]
NOMINAL_HBM_GBS = 8000.0
NOMINAL_BF16_TFLOPS = 2250.0
FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0}
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from `ncu` captures of one
# launch at the full workload size (profiles/): the gate-up GEMM at the 70B shape (512-row two-SM kernel) and at
# the 7B prefill shape (256-row two-SM kernel); small-batch kernel at M = 16 (the other small-batch sizes
# stream the same weights).
NCU_TRAFFIC_BYTES = {"c4_llama3_70b_prefill": 7219.9e6 + 469.0e6, "c2_llama2_7b_prefill": 238.98e6 + 82.55e6, "c3_llama3_8b_decode_m16": 357.20e6 + 4.04e6}
PARITY_REL_FRO = 5e-3
PARITY_SCALED_MAX_ABS = 8e-3


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def config_of(name, world):
    cfg = WORKLOADS[name]
    decode = name.startswith("c3_")
    return {"workload": name, "M": cfg["M"], "d": cfg["d"], "F": cfg["F"],
            "parallelism": "single GPU" if world == 1 else f"tp{world} (Megatron: gate/up column-split, down row-split)",
            "l2": ("no flush: four weight sets (1.4 GB) are cycled, every step streams from HBM" if decode else
                   "no flush: the per-step working set (weights + activations) exceeds the 126 MB L2")}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a timed region runs."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, index: int, period_s: float = 0.001):
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:  # noqa: BLE001
            self.nv = None

    def _loop(self):
        n = 0
        while not self._stop.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                if n % 8 == 0:
                    mask = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                    for bit, name in self.REASONS.items():
                        if mask & bit:
                            self.reasons.add(name)
            except Exception:  # noqa: BLE001
                pass
            n += 1
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        return False

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_mhz_min": min(self.samples),
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def flops_mlp(M, d, F):
    return 6.0 * M * d * F


# --------------------------------------------------------------------------- reference / CPU arm
def cpu_eager_sample(cfg, budget_s: float, steps: int | None, warmup: int):
    """Time the eager fp32 expression on a row slab at full d / F with all host threads."""
    from oracle import eager_reference as ref  # the checker, timed here as the CPU baseline

    torch.set_num_threads(os.cpu_count() or 1)
    d, F = cfg["d"], cfg["F"]
    g = torch.Generator().manual_seed(0)
    wg = torch.randn((F, d), generator=g) * 0.02
    wu = torch.randn((F, d), generator=g) * 0.02
    wd = torch.randn((d, F), generator=g) * 0.02
    rows = min(64, cfg["M"])
    x = torch.randn((rows, d), generator=g)
    ref.mlp_eager(x, wg, wu, wd)
    t0 = time.perf_counter()
    ref.mlp_eager(x, wg, wu, wd)
    t64 = time.perf_counter() - t0
    n_steps = steps if steps is not None else 10
    # the largest slab (<= 256 rows) that keeps the whole run inside the budget
    cands = [c for c in (256, 128, 64, 32, 16) if c <= cfg["M"]] or [cfg["M"]]
    for cand in cands:
        if t64 * cand / rows * (n_steps + warmup) <= budget_s or cand == cands[-1]:
            rows = cand
            break
    x = torch.randn((rows, d), generator=g)
    for _ in range(warmup):
        ref.mlp_eager(x, wg, wu, wd)
    ts = []
    for _ in range(n_steps):
        t0 = time.perf_counter()
        ref.mlp_eager(x, wg, wu, wd)
        ts.append(time.perf_counter() - t0)
    med = statistics.median(ts)
    return {"tflops": flops_mlp(rows, d, F) / med / 1e12, "rows": rows, "median_s": med, "total_s": sum(ts),
            "threads": torch.get_num_threads(), "steps": n_steps}


def run_reference(args, rank, world):
    if rank != 0:
        return
    name = args.workload or DEFAULT_WORKLOAD
    cfg = WORKLOADS[name]
    r = cpu_eager_sample(cfg, budget_s=150.0, steps=args.steps, warmup=args.warmup)
    sample = (f"eager fp32 (F.silu(x@Wg.T)*(x@Wu.T))@Wd.T on a {r['rows']}-row slab of {name} at full d/F, "
              f"{r['steps']} steps, median")
    line = {
        "impl": "reference", "metric": METRIC, "value": r["tflops"], "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["median_s"] * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_of(name, world), "sample_rows": r["rows"],
        "cpu_baseline": {"value": r["tflops"], "unit": UNIT, "cores": r["threads"], "kind": "port", "sample": sample},
        "e2e": {"value": r["tflops"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm: helpers
def vp(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def device_inputs(name, dev, world=1, rank=0, keep_full_on_host=False):
    """Seeded synthetic inputs generated on the device; the same bits on every rank.  Returns x, this
    rank's weight shard, and (optionally) the full weights as host tensors for the parity oracle."""
    import fused_swiglu_b200 as fsw

    cfg = WORKLOADS[name]
    M, d, F = cfg["M"], cfg["d"], cfg["F"]
    gx = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn((M, d), generator=gx, device=dev, dtype=torch.float32)
    if name.startswith("c5_"):
        mask = torch.rand((M, d), generator=gx, device=dev) < 0.01
        x = torch.where(mask, x * 50.0, x)
        del mask
    x = x.to(torch.bfloat16)
    lo, hi = fsw.pack.shard_bounds(F, world, rank)
    gw = torch.Generator(device=dev).manual_seed(1)
    shard, full_host = [], []
    for shape, axis in (((F, d), 0), ((F, d), 0), ((d, F), 1)):
        w = (torch.randn(shape, generator=gw, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        if keep_full_on_host:
            full_host.append(w.cpu())
        shard.append((w[lo:hi] if axis == 0 else w[:, lo:hi]).contiguous() if world > 1 else w)
        del w
    return x, shard, (full_host if keep_full_on_host else None)


def check_rows(M, n=40, seed=0):
    import numpy as np

    rng = np.random.default_rng(seed)
    edge = [r for r in (0, 1, 127, 128, 255, 256, M // 2, M - 257, M - 256, M - 129, M - 128, M - 2, M - 1) if 0 <= r < M]
    return sorted(set(edge + rng.choice(M, size=min(n, M), replace=False).tolist()))


def parity_record(out, x, full_host, world, dist_mod, dev):
    """Rows of `out` (all columns) against the fp32 expression on the CPU; identical bits on all ranks."""
    from oracle import swiglu_oracle as orc  # the checker

    rec = {}
    if world > 1:
        digest = torch.stack([out.view(torch.int16).to(torch.int64).sum(),
                              (out.view(torch.int16).to(torch.int64) * torch.arange(1, out.numel() + 1, device=dev)
                               .view_as(out) % 1000003).sum()])
        gathered = [torch.empty_like(digest) for _ in range(world)]
        dist_mod.all_gather(gathered, digest)
        rec["ranks_identical"] = all(torch.equal(g, digest) for g in gathered)
    if full_host is not None:
        f32 = lambda t: t.detach().float().cpu().numpy()  # noqa: E731
        rows = check_rows(out.size(0))
        ref = orc.mlp_fp32(f32(x[rows]), *[f32(w) for w in full_host])
        m = orc.error_metrics(f32(out[rows]), ref)
        rec.update({"rows_checked": len(rows), "rel_fro": m["rel_fro"], "max_abs": m["max_abs"],
                    "scaled_max_abs": m["scaled_max_abs"], "oracle": "fp32 expression on the CPU, same bf16 inputs",
                    "limits": {"rel_fro": PARITY_REL_FRO, "scaled_max_abs": PARITY_SCALED_MAX_ABS}})
    return rec


def kernel_name(M, n_out, K, gated):
    """Name of the tiled kernel the library takes for this problem (asked from the library itself)."""
    from fused_swiglu_b200 import capi
    which = int(capi.lib.fswiglu_plan_kernel(M, n_out, K, 1 if gated else 0))
    mode = "gated-split" if gated else "plain"
    return {0: f"gemm_tcgen05_kernel<{mode}> (one-SM tcgen05)",
            1: f"gemm_pair_kernel<{mode}> (two-SM tcgen05, cta_group::2, 256-row tiles)",
            2: f"gemm_quad_kernel<{mode}> (two-SM tcgen05, cta_group::2, 512-row tiles)"}.get(which, f"unknown ({which})")


def tensor_roofline(name, rows, d, Fl, gateup_ms, n_launches, region_ms, sms, world, clocks=None):
    """Denominator: the measured cuBLAS bf16 peak of the regime the timed region ran in - the burst figure
    while the GPU still boosts, the sustained one once the 1 kW power cap sets the clock (a region of
    half a second or more, or a median SM clock under 75 % of the maximum while it ran)."""
    peaks, peak_src = measured_peaks()
    capped = False
    if clocks and clocks.get("sm_mhz") and clocks.get("sm_max_mhz"):
        capped = clocks["sm_mhz"] < 0.75 * clocks["sm_max_mhz"]
    sustained = region_ms >= 500.0 or capped
    peak = peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"]
    flops = 4.0 * rows * d * Fl
    achieved = flops / (gateup_ms * 1e-3) / 1e12
    frac = achieved / peak
    assert frac <= 1.2, f"roofline fraction {frac:.2f} is not a measurement (flops and time of different launches?)"
    traffic = NCU_TRAFFIC_BYTES.get(name) if world == 1 else None
    return {"bound": "tensor", "kernel": kernel_name(rows, Fl, d, True) + ": gate-up + SiLU*up",
            "achieved": achieved, "peak": peak, "unit": UNIT, "frac": frac, "traffic": traffic,
            "peak_source": f"{peak_src} {'sustained' if sustained else 'burst'} cuBLAS bf16",
            "frac_of_burst_peak": achieved / peaks["bf16_tflops"],
            "frac_of_sustained_peak": achieved / peaks["bf16_tflops_sustained"],
            "frac_of_nominal_2250": achieved / NOMINAL_BF16_TFLOPS, "flops_per_launch": flops,
            "rows_per_launch": rows, "ms_per_launch": gateup_ms, "launches_timed": n_launches}


class SingleGpuPrefill:
    """Gate-up and down launches of one prefill workload on one GPU, with events around each launch."""

    def __init__(self, name, dev, stream, keep_full_on_host=False):
        import fused_swiglu_b200 as fsw
        from fused_swiglu_b200 import capi

        self.fsw, self.capi, self.lib = fsw, capi, capi.lib
        self.name, self.dev, self.stream = name, dev, stream
        cfg = WORKLOADS[name]
        self.M, self.d, self.F = cfg["M"], cfg["d"], cfg["F"]
        self.x, (self.wg, self.wu, self.wd), self.full_host = device_inputs(name, dev, keep_full_on_host=keep_full_on_host)
        self.h = torch.empty((self.M, self.F), dtype=torch.bfloat16, device=dev)
        self.out = torch.empty((self.M, self.d), dtype=torch.bfloat16, device=dev)
        self.scratch = fsw.ops.gemm_scratch(dev)
        self.sp = ctypes.c_void_p(stream.cuda_stream)
        self.events = []  # (gate-up begin, gate-up end = down begin, down end)

    def step(self, record):
        M, d, F, lib, sp = self.M, self.d, self.F, self.lib, self.sp
        if record:
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            ev[0].record(self.stream)
        rc = lib.fswiglu_gateup_bf16_ex(vp(self.x), d, vp(self.wg), d, vp(self.wu), vp(self.h), F, M, F, d, 0, None,
                                        vp(self.scratch), self.scratch.numel(), sp)
        if record:
            ev[1].record(self.stream)
        rc |= lib.fswiglu_down_bf16_ex(vp(self.h), F, vp(self.wd), F, vp(self.out), d, M, d, F, self.capi.OUT_BF16, None,
                                       0, vp(self.scratch), self.scratch.numel(), sp)
        if record:
            ev[2].record(self.stream)
            self.events.append(ev)
        self.capi.check(rc, "bench step")
        return self.out

    def kernel_ms(self):
        gu = statistics.mean(e[0].elapsed_time(e[1]) for e in self.events)
        dn = statistics.mean(e[1].elapsed_time(e[2]) for e in self.events)
        return gu, dn


def timed_region(step, steps, stream, sampler=None):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ctx = sampler if sampler is not None else _Null()
    with ctx:
        e0.record(stream)
        for _ in range(steps):
            step(True)
        e1.record(stream)
        torch.cuda.synchronize()
    return e0.elapsed_time(e1)


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def sustained_region(step, ms_per_step, stream, local_rank, min_seconds=2.0):
    """At least `min_seconds` of back-to-back steps: the clock-limited regime the short region does not reach."""
    n = max(20, int(min_seconds * 1e3 / max(ms_per_step, 1e-3)) + 1)
    sampler = ClockSampler(local_rank, period_s=0.001)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with sampler:
        e0.record(stream)
        for _ in range(n):
            step(False)
        e1.record(stream)
        torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n, n, sampler.summary()


def run_single_prefill(name, args, dev, stream, local_rank, with_parity, with_sustained):
    from fused_swiglu_b200 import capi

    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    w = SingleGpuPrefill(name, dev, stream, keep_full_on_host=with_parity)
    for _ in range(max(args.warmup, 3)):
        w.step(False)
    torch.cuda.synchronize()
    assert capi.device_status(stream.cuda_stream) == 0, "device watchdog tripped during warm-up"
    launches_before = capi.launch_count()
    sampler = ClockSampler(local_rank)
    total_ms = timed_region(w.step, args.steps, stream, sampler)
    launches = capi.launch_count() - launches_before
    assert capi.device_status(stream.cuda_stream) == 0, "device watchdog tripped during the timed region"
    ms = total_ms / args.steps
    gu_ms, dn_ms = w.kernel_ms()
    M, d, F = w.M, w.d, w.F
    rec = {"workload": name, "value": flops_mlp(M, d, F) / (ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms,
           "steps": args.steps, "tokens_per_s": M / (ms * 1e-3),
           "roofline": tensor_roofline(name, M, d, F, gu_ms, len(w.events), total_ms, sms, 1, sampler.summary()),
           "kernels": {"gate_up": {"kernel": kernel_name(M, F, d, True), "ms": gu_ms,
                                   "tflops": 4.0 * M * d * F / (gu_ms * 1e-3) / 1e12},
                       "down": {"kernel": kernel_name(M, d, F, False), "ms": dn_ms,
                                "tflops": 2.0 * M * d * F / (dn_ms * 1e-3) / 1e12}},
           "gpu_launches": int(launches), "clocks": sampler.summary()}
    clk = rec["clocks"].get("sm_mhz")
    if clk:
        rec["kernels"]["gate_up"]["ms_x_sm_mhz"] = gu_ms * clk
    if with_parity:
        rec["parity"] = parity_record(w.out, w.x, w.full_host, 1, None, dev)
    if with_sustained:
        s_ms, n, clocks = sustained_region(w.step, ms, stream, local_rank)
        peaks, _ = measured_peaks()
        val = flops_mlp(M, d, F) / (s_ms * 1e-3) / 1e12
        rec["sustained"] = {"value": val, "unit": UNIT, "ms_per_step": s_ms, "steps": n,
                            "frac_of_sustained_peak": val / peaks["bf16_tflops_sustained"],
                            "sm_mhz_median": clocks.get("sm_mhz"), "sm_mhz_min": clocks.get("sm_mhz_min"),
                            "samples": clocks["samples"], "reasons": clocks["reasons"]}
    return rec, w


def run_decode(name, args, dev, stream, local_rank, steps):
    """One cooperative weight-streaming kernel per step; four weight sets are cycled so that every step
    streams its 3*d*F*2 bytes from HBM (one set is 352 MB, L2 is 126 MB)."""
    import fused_swiglu_b200 as fsw
    from fused_swiglu_b200 import capi

    cfg = WORKLOADS[name]
    M, d, F = cfg["M"], cfg["d"], cfg["F"]
    x, first, _ = device_inputs(name, dev)
    gw = torch.Generator(device=dev).manual_seed(2)
    sets = [tuple(first)]
    for _ in range(3):
        sets.append(tuple((torch.randn(t.shape, generator=gw, device=dev) * 0.02).to(torch.bfloat16) for t in first))
    out = torch.empty((M, d), dtype=torch.bfloat16, device=dev)
    ws = fsw.ops.mlp_workspace(M, d, F, dev)
    sp = ctypes.c_void_p(stream.cuda_stream)
    events, counter = [], {"i": 0}

    def step(record):
        g_, u_, d_ = sets[counter["i"] % len(sets)]
        counter["i"] += 1
        if record:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
        rc = capi.lib.fswiglu_mlp_bf16(vp(x), d, vp(g_), vp(u_), d, vp(d_), F, vp(out), d, capi.OUT_BF16, M, d, F,
                                       vp(ws), ws.numel(), sp)
        if record:
            e1.record(stream)
            events.append((e0, e1))
        capi.check(rc, "bench decode step")

    for _ in range(max(args.warmup, 3) + 4):
        step(False)
    torch.cuda.synchronize()
    launches_before = capi.launch_count()
    sampler = ClockSampler(local_rank)
    total_ms = timed_region(step, steps, stream, sampler)
    launches = capi.launch_count() - launches_before
    assert capi.device_status(stream.cuda_stream) == 0, "device watchdog tripped (small-batch kernel)"
    ms = total_ms / steps
    launch_ms = statistics.mean(a.elapsed_time(b) for a, b in events)
    peaks, peak_src = measured_peaks()
    algo_bytes = 3.0 * d * F * 2 + 2.0 * M * d * 2
    gbs = algo_bytes / (launch_ms * 1e-3) / 1e9
    frac = gbs / peaks["hbm_gbs"]
    assert frac <= 1.2, "HBM roofline fraction above what the memory allows: not a measurement"
    return {"workload": name, "value": flops_mlp(M, d, F) / (ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms,
            "steps": steps, "tokens_per_s": M / (ms * 1e-3),
            "roofline": {"bound": "hbm", "kernel": "decode_fused_kernel (gate-up + SiLU*up + down, one launch)",
                         "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": frac,
                         "traffic": NCU_TRAFFIC_BYTES.get(name), "peak_source": f"{peak_src} copy bandwidth",
                         "frac_of_nominal_8000": gbs / NOMINAL_HBM_GBS, "bytes_per_launch": algo_bytes,
                         "ms_per_launch": launch_ms, "launches_timed": len(events)},
            "gpu_launches": int(launches), "clocks": sampler.summary()}


def run_backward(name, args, dev, stream, local_rank, steps):
    """Backward pass of one workload (16*M*d*F flops: seven GEMMs, two recomputing the pre-activations)."""
    import fused_swiglu_b200 as fsw
    from fused_swiglu_b200 import capi

    cfg = WORKLOADS[name]
    M, d, F = cfg["M"], cfg["d"], cfg["F"]
    x, (wg, wu, wd), _ = device_inputs(name, dev)
    dout = torch.randn((M, d), generator=torch.Generator(device=dev).manual_seed(3), device=dev).to(torch.bfloat16)
    ws = fsw.ops.backward_workspace(M, d, F, dev)
    grads = [torch.empty(shape, dtype=torch.bfloat16, device=dev) for shape in ((M, d), (F, d), (F, d), (d, F))]
    sp = ctypes.c_void_p(stream.cuda_stream)

    def step(record):
        rc = capi.lib.fswiglu_mlp_backward_bf16(vp(x), d, vp(wg), vp(wu), d, vp(wd), F, vp(dout), d, vp(grads[0]), d,
                                                vp(grads[1]), vp(grads[2]), d, vp(grads[3]), F, capi.OUT_BF16, M, d, F,
                                                vp(ws), ws.numel(), sp)
        capi.check(rc, "bench backward step")

    for _ in range(3):
        step(False)
    torch.cuda.synchronize()
    launches_before = capi.launch_count()
    sampler = ClockSampler(local_rank)
    total_ms = timed_region(step, steps, stream, sampler)
    launches = capi.launch_count() - launches_before
    assert capi.device_status(stream.cuda_stream) == 0, "device watchdog tripped (backward)"
    ms = total_ms / steps
    flops = 16.0 * M * d * F
    # spot check: dW_down rows against the chain rule evaluated with torch on the device in fp32
    h = (torch.nn.functional.silu(x.float() @ wg.float().T) * (x.float() @ wu.float().T))
    rows = torch.tensor([0, 1, d // 2, d - 1], device=dev)
    ref = dout.float().T[rows] @ h
    rel = float((grads[3][rows].float() - ref).norm() / ref.norm())
    assert rel <= 1e-2, f"backward spot check failed: {rel}"
    return {"workload": name.replace("prefill", "backward"), "value": flops / (ms * 1e-3) / 1e12, "unit": UNIT,
            "ms_per_step": ms, "steps": steps, "flops_per_step": flops,
            "what": "fswiglu_mlp_backward_bf16: dx, dW_gate, dW_up, dW_down in bf16 (7 GEMMs + 6 bandwidth-bound launches)",
            "rel_fro_dW_down_rows_vs_fp32": rel, "gpu_launches": int(launches), "clocks": sampler.summary()}


def e2e_single(w, args):
    """The same workload through the host-buffer entry point: x from pinned host memory, result back."""
    fsw = w.fsw
    M, d, F = w.M, w.d, w.F
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    x_host = w.x.cpu().pin_memory()
    out_host = torch.empty((M, d), dtype=torch.bfloat16).pin_memory()
    ws_host = fsw.ops.host_workspace(M, d, F, w.dev)
    for _ in range(3):
        fsw.ops.fused_swiglu_mlp_bf16_host(x_host, w.wg, w.wu, w.wd, out_host, ws_host)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        fsw.ops.fused_swiglu_mlp_bf16_host(x_host, w.wg, w.wu, w.wd, out_host, ws_host)
    torch.cuda.synchronize()
    s = (time.perf_counter() - t0) / e2e_steps
    # the host path works on 1024-row slabs, whose tiles are scheduled (and, in a split last wave, summed) differently
    # from the one-launch device path: same rounding points, results equal to within a bf16 ulp on a few entries
    dev_out = w.step(False).float()
    torch.cuda.synchronize()
    rel = float((out_host.to(w.dev).float() - dev_out).norm() / dev_out.norm())
    assert rel <= 1e-3, f"host-buffer path and device path disagree: rel-Fro {rel}"
    return {"value": flops_mlp(M, d, F) / s / 1e12, "unit": UNIT, "h2d_bytes_per_step": M * d * 2,
            "d2h_bytes_per_step": M * d * 2, "ms_per_step": s * 1e3, "steps": e2e_steps,
            "api": "fswiglu_mlp_bf16_host (row slabs pipelined over three streams)", "rel_fro_vs_device_path": rel}


def gpu_baselines(w, stream):
    """torch bf16 eager on the same GPU, and the reference's own kernel on its own benchmark problem."""
    import torch.nn.functional as Fn

    M, d, F = w.M, w.d, w.F
    rec = {}

    def eager():
        return (Fn.silu(w.x @ w.wg.T) * (w.x @ w.wu.T)) @ w.wd.T

    for _ in range(3):
        eager()
    torch.cuda.synchronize()
    ts = []
    for _ in range(8):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        eager()
        e1.record(stream)
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ms = statistics.median(ts)
    rec["torch_bf16_eager"] = {"workload": w.name, "ms_per_step": ms, "value": flops_mlp(M, d, F) / (ms * 1e-3) / 1e12,
                               "unit": UNIT, "what": "(F.silu(x@Wg.T)*(x@Wu.T))@Wd.T, bf16 tensors, cuBLAS + ATen kernels"}
    # the reference's benchmark problem: packed gate-up op, K = 8192, N = 2 * 28672, 4096 tokens
    Mb, K, N = 4096, 8192, 2 * 28672
    g = torch.Generator(device=w.dev).manual_seed(0)
    A = torch.randn((Mb, K), generator=g, device=w.dev, dtype=torch.float32).to(torch.bfloat16)
    B = (torch.randn((N, K), generator=g, device=w.dev, dtype=torch.float32) / K ** 0.5).to(torch.bfloat16)
    C = torch.zeros((Mb, N), dtype=torch.bfloat16, device=w.dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=w.dev)

    def ours():
        return w.lib.fswiglu_gateup_bf16_ex(vp(A), K, vp(B), K, None, vp(C), N // 2, Mb, N // 2, K, 1, None,
                                            vp(w.scratch), w.scratch.numel(), w.sp)

    for _ in range(3):
        w.capi.check(ours(), "legacy op")
    ts = []
    for _ in range(10):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        ours()
        e1.record(stream)
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ms = statistics.median(ts)
    rec["this_library_on_reference_problem"] = {
        "op": "swiglu_fwd_bf16 (packed W1W3)", "M": Mb, "K": K, "N": N, "ms": ms,
        "tflops": 2.0 * Mb * N * K / (ms * 1e-3) / 1e12, "l2": "256 MB buffer written between repetitions"}
    del A, B, C, flush
    torch.cuda.empty_cache()
    script = os.path.join(ROOT, "baseline", "ref_kernel_bench.py")
    try:
        res = subprocess.run([sys.executable, script, "--tokens", str(Mb)], capture_output=True, text=True, timeout=300)
        lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
        rec["reference_sm100a"] = json.loads(lines[-1]) if lines else {
            "unavailable": f"no result (exit {res.returncode}): {res.stderr.strip()[-160:]}"}
    except Exception as e:  # noqa: BLE001
        rec["reference_sm100a"] = {"unavailable": f"{type(e).__name__}: {str(e)[:120]}"}
    return rec


# --------------------------------------------------------------------------- GPU arm: one GPU
def run_one_gpu(args, local_rank):
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the SwiGLU path has no CPU fallback")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream(dev)
    name = args.workload or DEFAULT_WORKLOAD
    default_run = args.workload is None
    if name.startswith("c3_"):
        rec = run_decode(name, args, dev, stream, local_rank, args.steps)
        w = None
    else:
        rec, w = run_single_prefill(name, args, dev, stream, local_rank, with_parity=not args.no_parity,
                                    with_sustained=not args.no_sustained)
    line = {"metric": METRIC, "value": rec["value"], "unit": UNIT, "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": rec["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config_of(name, 1), "tokens_per_s": rec["tokens_per_s"],
            "frac_of_nominal_2250": rec["value"] / NOMINAL_BF16_TFLOPS,
            "roofline": rec["roofline"], "gpu_launches": rec["gpu_launches"], "clocks": rec["clocks"]}
    for k in ("kernels", "parity", "sustained"):
        if k in rec:
            line[k] = rec[k]
    if w is not None:
        line["e2e"] = e2e_single(w, args)
        if not args.no_gpu_baselines:
            line["gpu_baselines"] = gpu_baselines(w, stream)
    else:
        line["e2e"] = {"value": None, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                       "note": "small-batch workloads are reported device-resident only"}
    if "parity" in line and "rel_fro" in line["parity"]:
        p = line["parity"]
        assert p["rel_fro"] <= PARITY_REL_FRO and p["scaled_max_abs"] <= PARITY_SCALED_MAX_ABS, f"parity failed: {p}"
    del w
    torch.cuda.empty_cache()
    if default_run and not args.no_also:
        also = []
        sub = argparse.Namespace(**vars(args))
        for other in ALSO_AT_ONE_GPU:
            try:
                if other.startswith("c3_"):
                    also.append(run_decode(other, sub, dev, stream, local_rank, steps=max(args.steps, 200)))
                else:
                    sub.steps = max(args.steps, 50)
                    r, w2 = run_single_prefill(other, sub, dev, stream, local_rank, with_parity=not args.no_parity,
                                               with_sustained=False)
                    also.append(r)
                    del w2
            except Exception as e:  # noqa: BLE001  (a sub-record must not take the headline down with it)
                also.append({"workload": other, "error": f"{type(e).__name__}: {str(e)[:200]}"})
            torch.cuda.empty_cache()
        try:
            also.append(run_backward("c2_llama2_7b_prefill", sub, dev, stream, local_rank, steps=max(args.steps, 20)))
        except Exception as e:  # noqa: BLE001
            also.append({"workload": "c2_llama2_7b_backward", "error": f"{type(e).__name__}: {str(e)[:200]}"})
        torch.cuda.empty_cache()
        line["also"] = also
    if not args.no_cpu_baseline:
        r = cpu_eager_sample(WORKLOADS[name], budget_s=20.0, steps=None, warmup=1)
        line["cpu_baseline"] = {
            "value": r["tflops"], "unit": UNIT, "cores": r["threads"], "kind": "port",
            "sample": f"eager fp32 expression on a {r['rows']}-row slab of {name} at full d/F, "
                      f"{r['steps']} runs, median {r['median_s'] * 1e3:.1f} ms"}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm: tensor parallel
def run_tensor_parallel(args, rank, local_rank, world):
    import torch.distributed as dist

    from fused_swiglu_b200 import capi
    from fused_swiglu_b200.tp import TensorParallelSwiGLU

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the SwiGLU path has no CPU fallback")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    # NCCL collectives that run beside persistent GEMMs are capped to the SMs the GEMMs leave free
    os.environ.setdefault("NCCL_MAX_CTAS", str(max(args.comm_sms, 8)))
    dist.init_process_group("nccl", device_id=dev)
    name = args.workload or DEFAULT_WORKLOAD
    if name.startswith("c3_"):
        raise SystemExit("the small-batch workloads are single-GPU")
    if args.tp_mode != "push" and args.comm_sms == 0:
        args.comm_sms = 16  # NCCL kernels cannot share an SM with a persistent GEMM CTA: set SMs aside for them
    cfg = WORKLOADS[name]
    M, d, F = cfg["M"], cfg["d"], cfg["F"]
    want_parity = not args.no_parity
    x, (wg, wu, wd), full_host = device_inputs(name, dev, world, rank, keep_full_on_host=want_parity and rank == 0)
    Fl = wg.size(0)
    stream = torch.cuda.current_stream(dev)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count

    tp = TensorParallelSwiGLU(wg, wu, wd, n_slabs=args.slabs, mode=args.tp_mode, comm_sms=args.comm_sms,
                              reduce_ctas=args.reduce_ctas,
                              slab_rows=[int(v) for v in args.slab_rows.split(",")] if args.slab_rows else None)
    bounds = tp.slab_bounds(M)
    trace_log, recording = [], {"on": False}

    def trace(tag, slab, on_stream):
        if recording["on"]:
            e = torch.cuda.Event(enable_timing=True)
            e.record(on_stream)
            trace_log.append((tag, slab, e))
    tp.trace = trace

    def step(record):
        recording["on"] = record
        return tp.forward(x)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(max(args.warmup, 3)):
        step(False)
    barrier()
    assert capi.device_status(stream.cuda_stream) == 0, "device watchdog tripped during warm-up"
    launches_before = capi.launch_count()
    ev_start, ev_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local_rank)
    barrier()
    with sampler:
        ev_start.record(stream)
        for _ in range(args.steps):
            out = step(True)
        ev_end.record(stream)
        barrier()
    total_ms = ev_start.elapsed_time(ev_end)
    launches = capi.launch_count() - launches_before
    t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    value = flops_mlp(M, d, F) / (ms_per_step * 1e-3) / 1e12
    assert capi.device_status(stream.cuda_stream) == 0, "device watchdog tripped during the timed region"
    recording["on"] = False

    # per-phase timeline (this rank): mean duration between consecutive marks, per slab
    timeline, gateup_by_slab = {}, {}
    marks = {}
    for tag, slab, e in trace_log:
        marks.setdefault((slab, tag), []).append(e)
    order = ["gateup_begin", "gateup_end", "down_end", "barrier_end", "reduce_end"]
    for si in range(len(bounds)):
        for a, b in zip(order, order[1:]):
            ea, eb = marks.get((si, a)), marks.get((si, b))
            if ea and eb and len(ea) == len(eb):
                timeline[f"slab{si}:{a}->{b}"] = statistics.mean(p.elapsed_time(q) for p, q in zip(ea, eb))
        if (si, "gateup_begin") in marks and (si, "gateup_end") in marks:
            gateup_by_slab[si] = timeline.get(f"slab{si}:gateup_begin->gateup_end")
    fin_a, fin_b = marks.get((len(bounds) - 1, "reduce_end")), marks.get((-1, "final_barrier_end"))
    if fin_a and fin_b and len(fin_a) == len(fin_b):
        timeline["last_reduce_end->final_barrier_end"] = statistics.mean(p.elapsed_time(q) for p, q in zip(fin_a, fin_b))

    parity = parity_record(out, x, full_host, world, dist, dev) if want_parity else None

    # ----------------------------- end to end through host buffers -------------------------------
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    x_host = x.cpu().pin_memory()
    out_host = torch.empty((sum(g1 - g0 for g0, g1 in tp.owned_rows(M)), d), dtype=torch.bfloat16).pin_memory()
    for _ in range(3):
        tp.forward_from_host(x_host, out_host)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        tp.forward_from_host(x_host, out_host)
    barrier()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    t = torch.tensor([e2e_s], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_s = float(t.item())
    h2d = M * d * 2 if args.tp_mode == "push" else M * d * 2 * world

    if rank == 0:
        # roofline of the gate-up launch of the tallest slab: its own flops over its own time
        tall = max(range(len(bounds)), key=lambda i: bounds[i][1] - bounds[i][0])
        rows = bounds[tall][1] - bounds[tall][0]
        gu_ms = gateup_by_slab.get(tall)
        roofline = (tensor_roofline(name, rows, d, Fl, gu_ms, len(marks.get((tall, "gateup_begin"), [])), total_ms, sms,
                                    world, sampler.summary()) if gu_ms else None)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config_of(name, world), "tokens_per_s": M / (ms_per_step * 1e-3),
            "frac_of_nominal_2250_per_gpu": value / world / NOMINAL_BF16_TFLOPS,
            "tp": {"mode": args.tp_mode, "slab_rows": [b - a for a, b in bounds], "comm_sms": args.comm_sms,
                   "reduce_ctas": args.reduce_ctas, "timeline_ms_rank0": timeline},
            "roofline": roofline,
            "e2e": {"value": flops_mlp(M, d, F) / e2e_s / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": M * d * 2, "ms_per_step": e2e_s * 1e3, "steps": e2e_steps,
                    "api": "TensorParallelSwiGLU.forward_from_host (1/N of x over PCIe per rank, rest over NVLink; copies of slab i+1 and of the finished rows of slab i-1 overlap the GEMMs of slab i)"},
            "gpu_launches": int(launches), "clocks": sampler.summary(),
        }
        if parity is not None:
            line["parity"] = parity
        print(json.dumps(line), flush=True)
        if parity is not None:
            assert parity.get("ranks_identical", True), "ranks hold different results"
            if "rel_fro" in parity:
                assert parity["rel_fro"] <= PARITY_REL_FRO and parity["scaled_max_abs"] <= PARITY_SCALED_MAX_ABS, parity
    dist.barrier()
    tp.close()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default=None)
    ap.add_argument("--e2e-steps", type=int, default=50)
    ap.add_argument("--slabs", type=int, default=0, help="row slabs per step when N > 1 (0: planned from a cost model)")
    ap.add_argument("--tp-mode", choices=["allreduce", "rs_ag", "push"], default="push")
    ap.add_argument("--comm-sms", type=int, default=0,
                    help="SMs withheld from the GEMMs for communication kernels when N > 1 (push mode needs none)")
    ap.add_argument("--reduce-ctas", type=int, default=128, help="CTAs of the reduce+broadcast kernel (push mode)")
    ap.add_argument("--slab-rows", type=str, default="", help="explicit slab heights, e.g. 3840,3840,512")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-gpu-baselines", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--no-sustained", action="store_true")
    ap.add_argument("--no-also", action="store_true", help="skip the c2 / c3 sub-records of the default one-GPU run")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world == 1 and args.gpus > 1:
        raise SystemExit(f"--gpus {args.gpus} needs one process per GPU: launch with "
                         f"python -m torch.distributed.run --nnodes=1 --nproc-per-node {args.gpus} "
                         f"--master-addr 127.0.0.1 --master-port 29500 bench.py --gpus {args.gpus} ...")
    if args.impl == "reference":
        run_reference(args, rank, world)
    elif world == 1:
        run_one_gpu(args, local_rank)
    else:
        run_tensor_parallel(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
