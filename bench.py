#!/usr/bin/env python
"""Benchmark of the fused SwiGLU MLP forward on B200: `python bench.py --gpus N --steps K --warmup W`.

One "step" is one forward pass out = (silu(x Wg^T) * (x Wu^T)) Wd^T over one batch of synthetic
bf16 input (x ~ N(0,1), weights ~ N(0, 0.02^2), seeded).

  N = 1   workload c2: Llama-2-7B MLP prefill, M=4096, d=4096, F=11008, single B200.
  N > 1   workload c4: Llama-3-70B MLP prefill, M=8192, d=8192, F=28672, Megatron tensor-parallel over
          the N ranks (W_gate/W_up column-split, W_down row-split, fp32 all-reduce of the output):
          total work is fixed as N grows ("scaling": "strong").  Launch with torchrun, one rank per GPU.

The JSON line printed by rank 0 carries
  value     whole-job TFLOP/s (6*M*d*F flops per step) with inputs resident in HBM, timed with CUDA
            events on the launching stream over exactly K steps, max over ranks;
  e2e       the same metric through the host-buffer entry point: every step copies x from pinned host
            memory to the device and the result back, inside the timed region;
  roofline  of the dominant kernel (the gate-up tcgen05 GEMM, two thirds of the flops): algorithmic
            flops per launch / its mean launch duration (CUDA events around each launch inside the timed
            region) against the measured dense-bf16 peak in MEASURED_PEAKS.json;
  cpu_baseline  (N = 1) the eager PyTorch expression in fp32 on this box's host cores, on a row slab.

`--impl reference` times only that CPU expression (the reference project's own oracle arithmetic;
its CUDA kernel covers the gate-up half only and has no sm_100 build) and prints the same line shape.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "fused-swiglu_b200"))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "fused SwiGLU MLP fwd TFLOP/s"
UNIT = "TFLOP/s"
WORKLOADS = {
    "c2_llama2_7b_prefill": dict(M=4096, d=4096, F=11008),
    "c4_llama3_70b_prefill": dict(M=8192, d=8192, F=28672),
    # small-batch (HBM-bound) configurations: single GPU only, roofline = HBM bandwidth
    "c3_llama3_8b_decode_m1": dict(M=1, d=4096, F=14336),
    "c3_llama3_8b_decode_m4": dict(M=4, d=4096, F=14336),
    "c3_llama3_8b_decode_m16": dict(M=16, d=4096, F=14336),
    "c3_llama3_8b_decode_m64": dict(M=64, d=4096, F=14336),
}
NOMINAL_HBM_GBS = 8000.0
NOMINAL_BF16_TFLOPS = 2250.0
FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0}
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from `ncu --set full`
# captures of one launch at the full workload size (two-SM gate-up GEMM at the 7B prefill shape; small-batch
# kernel at M = 16; the other small-batch sizes stream the same weights).
NCU_TRAFFIC_BYTES = {"c2_llama2_7b_prefill": 238.52e6 + 82.92e6, "c4_llama3_70b_prefill": None,
                     "c3_llama3_8b_decode_m16": 353.64e6 + 3.78e6}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return p, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, index: int, period_s: float = 0.01):
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
        while not self._stop.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                mask = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:  # noqa: BLE001
                pass
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
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


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
    rows = 64
    x = torch.randn((rows, d), generator=g)
    ref.mlp_eager(x, wg, wu, wd)
    t0 = time.perf_counter()
    ref.mlp_eager(x, wg, wu, wd)
    t64 = time.perf_counter() - t0
    n_steps = steps if steps is not None else 10
    # the largest slab (<= 256 rows) that keeps the whole run inside the budget
    cands = [c for c in (256, 128, 64, 32, 16) if c <= cfg["M"]] or [cfg["M"]]
    for cand in cands:
        if t64 * cand / 64 * (n_steps + warmup) <= budget_s or cand == cands[-1]:
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
    name = "c2_llama2_7b_prefill" if world == 1 else "c4_llama3_70b_prefill"
    cfg = WORKLOADS[name]
    r = cpu_eager_sample(cfg, budget_s=150.0, steps=args.steps, warmup=args.warmup)
    sample = (f"eager fp32 (F.silu(x@Wg.T)*(x@Wu.T))@Wd.T on a {r['rows']}-row slab of {name} at full d/F, "
              f"{r['steps']} steps, median")
    line = {
        "impl": "reference", "metric": METRIC, "value": r["tflops"], "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["median_s"] * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, **cfg, "sample_rows": r["rows"]},
        "cpu_baseline": {"value": r["tflops"], "unit": UNIT, "cores": r["threads"], "kind": "port", "sample": sample},
        "e2e": {"value": r["tflops"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm
def vp(t):
    return ctypes.c_void_p(t.data_ptr())


def run_ours(args, rank, local_rank, world):
    import torch.distributed as dist

    import fused_swiglu_b200 as fsw
    from fused_swiglu_b200 import capi
    from fused_swiglu_b200.tp import TensorParallelSwiGLU

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the SwiGLU path has no CPU fallback")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        # the collectives run beside persistent GEMMs: cap NCCL's CTAs to the SMs the GEMMs leave free
        os.environ.setdefault("NCCL_MAX_CTAS", str(args.comm_sms))
        dist.init_process_group("nccl", device_id=dev)
    name = args.workload or ("c2_llama2_7b_prefill" if world == 1 else "c4_llama3_70b_prefill")
    cfg = WORKLOADS[name]
    M, d, F = cfg["M"], cfg["d"], cfg["F"]
    lo, hi = fsw.pack.shard_bounds(F, world, rank)
    Fl = hi - lo

    # synthetic inputs, generated on the device: x is the same on every rank, weights are the rank's shard
    gx = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn((M, d), generator=gx, device=dev, dtype=torch.float32).to(torch.bfloat16)
    gw = torch.Generator(device=dev).manual_seed(1000 + rank)
    wg = (torch.randn((Fl, d), generator=gw, device=dev) * 0.02).to(torch.bfloat16)
    wu = (torch.randn((Fl, d), generator=gw, device=dev) * 0.02).to(torch.bfloat16)
    wd = (torch.randn((d, Fl), generator=gw, device=dev) * 0.02).to(torch.bfloat16)
    stream = torch.cuda.current_stream(dev)
    sp = ctypes.c_void_p(stream.cuda_stream)
    lib = capi.lib
    gateup_events = []

    decode = name.startswith("c3_")
    if decode and world > 1:
        raise SystemExit("the small-batch workloads are single-GPU")
    if decode:
        # one cooperative weight-streaming kernel per step; four weight sets are cycled so that every
        # step streams its 3*d*F*2 bytes from HBM (one set is 352 MB, L2 is 126 MB)
        n_sets = 4
        sets = [(wg, wu, wd)]
        for _ in range(n_sets - 1):
            sets.append(tuple((torch.randn(t.shape, generator=gw, device=dev) * 0.02).to(torch.bfloat16)
                              for t in (wg, wu, wd)))
        out = torch.empty((M, d), dtype=torch.bfloat16, device=dev)
        ws_dec = fsw.ops.mlp_workspace(M, d, F, dev)
        counter = {"i": 0}

        def step(record):
            g_, u_, d_ = sets[counter["i"] % n_sets]
            counter["i"] += 1
            if record:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
            rc = lib.fswiglu_mlp_bf16(vp(x), d, vp(g_), vp(u_), d, vp(d_), F, vp(out), d, capi.OUT_BF16, M, d, F,
                                      vp(ws_dec), ws_dec.numel(), sp)
            if record:
                e1.record(stream)
                gateup_events.append((e0, e1))
            capi.check(rc, "bench decode step")
            return out
        gateup_rows = M
        parallelism = "single GPU, small-batch weight-streaming kernel"
    elif world == 1:
        h = torch.empty((M, F), dtype=torch.bfloat16, device=dev)
        out = torch.empty((M, d), dtype=torch.bfloat16, device=dev)

        def step(record):
            if record:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
            rc = lib.fswiglu_gateup_bf16(vp(x), d, vp(wg), d, vp(wu), vp(h), F, M, F, d, 0, sp)
            if record:
                e1.record(stream)
                gateup_events.append((e0, e1))
            rc |= lib.fswiglu_down_bf16(vp(h), F, vp(wd), F, vp(out), d, M, d, F, capi.OUT_BF16, sp)
            capi.check(rc, "bench step")
            return out
        gateup_rows = M
        parallelism = "single GPU"
    else:
        record_flag = {"on": False}

        def local_partial(xs, g_, u_, dn_, out_f32, ws):
            rows = xs.size(0)
            hbuf = ws[: rows * Fl * 2].view(torch.bfloat16).view(rows, Fl)
            if record_flag["on"]:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
            rc = lib.fswiglu_gateup_bf16(vp(xs), d, vp(g_), d, vp(u_), vp(hbuf), Fl, rows, Fl, d, 0, sp)
            if record_flag["on"]:
                e1.record(stream)
                gateup_events.append((e0, e1))
            rc |= lib.fswiglu_down_bf16(vp(hbuf), Fl, vp(dn_), Fl, vp(out_f32), d, rows, d, Fl, capi.OUT_F32, sp)
            capi.check(rc, "bench tp step")

        tp = TensorParallelSwiGLU(wg, wu, wd, n_slabs=args.slabs, mode=args.tp_mode, local_partial=local_partial,
                                  comm_sms=args.comm_sms, reduce_ctas=args.reduce_ctas,
                                  slab_rows=[int(v) for v in args.slab_rows.split(",")] if args.slab_rows else None)
        gateup_rows = max(r1 - r0 for r0, r1 in tp.slab_bounds(M))
        pending = []

        def trace(tag):
            if not record_flag["on"]:
                return
            e = torch.cuda.Event(enable_timing=True)
            e.record(stream)
            if tag == "gateup_begin":
                pending.append(e)
            else:
                gateup_events.append((pending.pop(), e))
        tp.trace = trace

        def step(record):
            record_flag["on"] = record
            return tp.forward(x)
        parallelism = f"tp{world} (Megatron: gate/up column-split, down row-split, {args.tp_mode}, " \
                      f"{len(tp.slab_bounds(M))} row slabs overlapped)"

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(max(args.warmup, 3)):
        step(False)
    barrier()
    assert capi.device_status(stream.cuda_stream) == 0, "device watchdog tripped during warm-up"

    # ----------------------------- timed region: exactly K steps ---------------------------------
    launches_before = capi.launch_count()
    ev_start, ev_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local_rank)
    barrier()
    with sampler:
        ev_start.record(stream)
        for _ in range(args.steps):
            step(True)
        ev_end.record(stream)
        barrier()
    total_ms = ev_start.elapsed_time(ev_end)
    launches = capi.launch_count() - launches_before
    if world > 1:
        t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    value = flops_mlp(M, d, F) / (ms_per_step * 1e-3) / 1e12
    gateup_ms = statistics.mean(a.elapsed_time(b) for a, b in gateup_events)
    assert capi.device_status(stream.cuda_stream) == 0, "device watchdog tripped during the timed region"

    # ----------------------------- end to end through host buffers -------------------------------
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    x_host = x.cpu().pin_memory()
    if world == 1:
        out_host = torch.empty((M, d), dtype=torch.bfloat16).pin_memory()
        ws_host = fsw.ops.host_workspace(M, d, F, dev)

        def e2e_step():
            fsw.ops.fused_swiglu_mlp_bf16_host(x_host, wg, wu, wd, out_host, ws_host)
        h2d, d2h = M * d * 2, M * d * 2
    else:
        rows_per = (M + world - 1) // world
        r0, r1 = min(M, rank * rows_per), min(M, (rank + 1) * rows_per)
        out_host = torch.empty((r1 - r0, d), dtype=torch.bfloat16).pin_memory()

        def e2e_step():
            tp.trace = None
            tp.forward_from_host(x_host, out_host)
        # per step: every rank reads its 1/world slice of x from the host and writes its slice of out
        h2d, d2h = (M * d * 2 if args.tp_mode == "push" else M * d * 2 * world), M * d * 2
    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_s], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_value = flops_mlp(M, d, F) / e2e_s / 1e12

    if rank == 0:
        peaks, peak_src = measured_peaks()
        long_region = total_ms >= 500.0
        peak = peaks["bf16_tflops_sustained"] if long_region else peaks["bf16_tflops"]
        gateup_flops = 4.0 * gateup_rows * d * Fl
        achieved = gateup_flops / (gateup_ms * 1e-3) / 1e12
        traffic = NCU_TRAFFIC_BYTES.get(name)
        if traffic is not None and world > 1:
            traffic = None  # captured for the single-GPU shape only
        if decode:
            algo_bytes = 3.0 * d * F * 2 + 2.0 * M * d * 2
            hbm_peak = peaks["hbm_gbs"]
            hbm_achieved = algo_bytes / (gateup_ms * 1e-3) / 1e9
            roofline = {"bound": "hbm", "kernel": "decode_fused_kernel (gate-up + SiLU*up + down, one launch)",
                        "achieved": hbm_achieved, "peak": hbm_peak, "unit": "GB/s", "frac": hbm_achieved / hbm_peak,
                        "traffic": traffic, "peak_source": f"{peak_src} copy bandwidth",
                        "frac_of_nominal_8000": hbm_achieved / NOMINAL_HBM_GBS, "bytes_per_launch": algo_bytes,
                        "ms_per_launch": gateup_ms, "launches_timed": len(gateup_events)}
        else:
            roofline = {"bound": "tensor", "kernel": "gemm_pair_kernel<gated-split> (gate-up + SiLU*up, two-SM tcgen05)",
                        "achieved": achieved, "peak": peak, "unit": UNIT, "frac": achieved / peak,
                        "traffic": traffic, "peak_source": f"{peak_src} {'sustained' if long_region else 'burst'}",
                        "flops_per_launch": gateup_flops, "ms_per_launch": gateup_ms,
                        "launches_timed": len(gateup_events)}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": name, "M": M, "d": d, "F": F, "parallelism": parallelism,
                       "l2": ("no flush: four weight sets (1.4 GB) are cycled, every step streams from HBM" if decode else
                              "no flush: per-step working set (weights + activations) exceeds the 126 MB L2"),
                       "tokens_per_s": M / (ms_per_step * 1e-3),
                       "frac_of_nominal_2250": value / world / NOMINAL_BF16_TFLOPS,
                       "frac_of_measured_peak": value / world / peak},
            "roofline": roofline,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_s * 1e3, "steps": e2e_steps},
            "gpu_launches": int(launches),
            "clocks": sampler.summary(),
        }
        if world == 1 and not args.no_cpu_baseline:
            r = cpu_eager_sample(cfg, budget_s=20.0, steps=None, warmup=1)
            line["cpu_baseline"] = {
                "value": r["tflops"], "unit": UNIT, "cores": r["threads"], "kind": "port",
                "sample": f"eager fp32 expression on a {r['rows']}-row slab of {name} at full d/F, "
                          f"{r['steps']} runs, median {r['median_s'] * 1e3:.1f} ms"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default=None)
    ap.add_argument("--e2e-steps", type=int, default=50)
    ap.add_argument("--slabs", type=int, default=0, help="row slabs per step when N > 1 (0: planned from a cost model)")
    ap.add_argument("--tp-mode", choices=["allreduce", "rs_ag", "push"], default="push")
    ap.add_argument("--comm-sms", type=int, default=16, help="SMs left to the collective kernels when N > 1")
    ap.add_argument("--reduce-ctas", type=int, default=32, help="CTAs of the reduce+broadcast kernel (0: = comm-sms)")
    ap.add_argument("--slab-rows", type=str, default="", help="explicit slab heights, e.g. 3840,3840,512")
    ap.add_argument("--no-cpu-baseline", action="store_true")
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
    else:
        run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
