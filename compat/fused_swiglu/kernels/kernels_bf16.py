"""Stand-in for fused_swiglu.kernels.kernels_bf16: only the name bench_swiglu.py:9 imports."""


def fused_swiglu_fwd(*args, **kwargs):
    raise NotImplementedError("fused_swiglu (fattorib) is not installed; this is an import-only stand-in")
