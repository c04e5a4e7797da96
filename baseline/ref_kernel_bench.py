"""Time the reference project's own kernel (rebuilt for sm_100a by build_ref_kernel.py) on its own
benchmark problem: the packed gate-up op at K = 8192, N = 2 * 28672 (bench_swiglu.py:84-91,106 of
the reference), through its own binding swiglu_fwd_bf16(M, N, K, A, K, B, K, C, N).

Runs in a process of its own (bench.py starts it): the module registers the same dispatcher
namespace as this repository's extension, so the two are never loaded together, and none of this
repository's kernels is on this path.  Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--n", type=int, default=2 * 28672)
    ap.add_argument("--reps", type=int, default=10)
    a = ap.parse_args()
    sys.path.insert(0, os.path.join(HERE, "_ref"))
    try:
        import torch
        import fused_mlp_module_ref as ref
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"unavailable": f"reference kernel module not importable: {type(e).__name__}: {str(e)[:120]}"}))
        return
    if not torch.cuda.is_available():
        print(json.dumps({"unavailable": "no CUDA device"}))
        return
    M, K, N = a.tokens, a.k, a.n
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(0)
    A = torch.randn((M, K), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    B = (torch.randn((N, K), generator=g, device=dev, dtype=torch.float32) / K ** 0.5).to(torch.bfloat16)
    C = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # larger than the 126 MB L2
    for _ in range(3):
        ref.swiglu_fwd_bf16(M, N, K, A, K, B, K, C, N)
    torch.cuda.synchronize()
    times = []
    for _ in range(a.reps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ref.swiglu_fwd_bf16(M, N, K, A, K, B, K, C, N)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    ms = times[len(times) // 2]
    # row sample against an fp32 computation on the same device (sanity of the rebuilt kernel, not a parity claim)
    rows = torch.tensor([0, 1, 255, 256, M - 1], device=dev)
    acc = A[rows].float() @ B.float().T
    want = acc[:, 0::2] * torch.nn.functional.silu(acc[:, 1::2])
    got = C.flatten()[: M * N // 2].view(M, N // 2)[rows].float()
    rel = float((got - want).norm() / want.norm())
    print(json.dumps({"kernel": "Fused_MLP::gemm_device (reference, mma.sync, rebuilt for sm_100a)", "M": M, "K": K, "N": N,
                      "ms": ms, "tflops": 2.0 * M * N * K / (ms * 1e-3) / 1e12, "reps": a.reps,
                      "rel_fro_vs_fp32_rows": rel, "l2": "256 MB buffer written between repetitions"}))


if __name__ == "__main__":
    main()
