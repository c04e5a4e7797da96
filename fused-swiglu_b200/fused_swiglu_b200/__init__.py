"""B200 (sm_100a) fused SwiGLU MLP forward: Python host layer over libfswiglu.so.

    ops     the reference's operator surface (fused_swiglu_bf16, swiglu_fwd_bf16) plus the
            split-weight, down-projection and whole-MLP ops, all through the C ABI
    capi    ctypes binding of include/fswiglu.h
    pack    interleaved <-> split weight layouts, tensor-parallel shards
    tp      Megatron-style tensor-parallel forward (one process per GPU, NCCL)
    inputs  seeded synthetic inputs of the benchmark configurations
    module  nn.Module wrapper (gate_proj / up_proj / down_proj) over the dispatcher op

Importing the package loads the CUDA library and raises if it has not been built.
"""
from . import capi, inputs, ops, pack  # noqa: F401
from .ops import (  # noqa: F401
    fused_swiglu_bf16,
    fused_swiglu_gateup_bf16,
    fused_swiglu_mlp_bf16,
    fused_swiglu_mlp_bf16_host,
    swiglu_down_bf16,
    swiglu_fwd_bf16,
)

__version__ = capi.version()
