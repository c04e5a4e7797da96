"""cuBLAS (torch.matmul) on the two GEMM shapes of a workload, a few launches each.

A GPU baseline for profiling, not part of the product path: run it under an ncu metrics pass to read what the
vendor library moves through L2 and HBM, and how busy it keeps the tensor pipe, on the shapes the library's own
kernels are profiled on.  The gate-up GEMM is x [M, d] times the stacked [W_gate; W_up] [2F, d] (no SiLU, both
halves written); the down GEMM is h [M, F] times W_down [d, F].

    python baseline/cublas_gemm_shapes.py [M d F] [gu|dn|both]        (default: 8192 8192 28672 both)
"""
import sys

import torch


def main() -> None:
    args = [a for a in sys.argv[1:]]
    which = "both"
    if args and args[-1] in ("gu", "dn", "both"):
        which = args.pop()
    M, d, F = (int(v) for v in args[:3]) if len(args) >= 3 else (8192, 8192, 28672)
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(0)

    def rnd(rows, cols, scale):
        return (torch.randn((rows, cols), device=dev, generator=g) * scale).to(torch.bfloat16)

    if which in ("gu", "both"):
        x, w = rnd(M, d, 1.0), rnd(2 * F, d, 0.02)
        for _ in range(3):
            c = x @ w.t()
        torch.cuda.synchronize()
        del x, w, c
    if which in ("dn", "both"):
        h, wd = rnd(M, F, 1.0), rnd(d, F, 0.02)
        for _ in range(3):
            o = h @ wd.t()
        torch.cuda.synchronize()
        del h, wd, o
    print(f"cuBLAS GEMM shapes M={M} d={d} F={F} ({which}): done")


if __name__ == "__main__":
    main()
