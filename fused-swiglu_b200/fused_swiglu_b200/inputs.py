"""Seeded synthetic inputs for the five benchmark configurations.

Shapes are the MLP dimensions of Llama-2-7B/13B and Llama-3-8B/70B; values are drawn on
the CPU with torch.Generator().manual_seed(seed) in the fixed order x, W_gate, W_up,
W_down (fp32), scaled, and rounded to bf16, so a CPU checker and the GPU see identical
bits.  x ~ N(0,1); weights ~ N(0, 0.02^2).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class MlpConfig:
    name: str
    M: int
    d: int
    F: int
    tp: int = 1
    ragged: bool = False


CONFIGS = {
    "c1_cpu_small": MlpConfig("c1_cpu_small", 512, 1024, 2816),
    "c2_llama2_7b_prefill": MlpConfig("c2_llama2_7b_prefill", 4096, 4096, 11008),
    "c3_llama3_8b_decode_m1": MlpConfig("c3_llama3_8b_decode_m1", 1, 4096, 14336),
    "c3_llama3_8b_decode_m4": MlpConfig("c3_llama3_8b_decode_m4", 4, 4096, 14336),
    "c3_llama3_8b_decode_m16": MlpConfig("c3_llama3_8b_decode_m16", 16, 4096, 14336),
    "c3_llama3_8b_decode_m64": MlpConfig("c3_llama3_8b_decode_m64", 64, 4096, 14336),
    "c4_llama3_70b_prefill": MlpConfig("c4_llama3_70b_prefill", 8192, 8192, 28672, tp=8),
    "c5_ragged_13b": MlpConfig("c5_ragged_13b", -1, 5120, 13824, tp=8, ragged=True),
}

WEIGHT_STD = 0.02


def ragged_lengths(seed: int = 0, n_seq: int = 32, max_len: int = 2048) -> torch.Tensor:
    """Sequence lengths of the ragged-batch stress case: uniform in [1, max_len]."""
    g = torch.Generator().manual_seed(seed)
    return torch.randint(1, max_len + 1, (n_seq,), generator=g)


def make_x(M: int, d: int, g: torch.Generator, outliers: bool = False) -> torch.Tensor:
    x = torch.randn((M, d), generator=g, dtype=torch.float32)
    if outliers:
        mask = torch.rand((M, d), generator=g) < 0.01
        x = torch.where(mask, x * 50.0, x)
    return x.to(torch.bfloat16)


def make_weights(d: int, F: int, g: torch.Generator):
    w_gate = (torch.randn((F, d), generator=g, dtype=torch.float32) * WEIGHT_STD).to(torch.bfloat16)
    w_up = (torch.randn((F, d), generator=g, dtype=torch.float32) * WEIGHT_STD).to(torch.bfloat16)
    w_down = (torch.randn((d, F), generator=g, dtype=torch.float32) * WEIGHT_STD).to(torch.bfloat16)
    return w_gate, w_up, w_down


def make_mlp_inputs(M: int, d: int, F: int, seed: int = 0, outliers: bool = False):
    """(x, W_gate, W_up, W_down) as bf16 CPU tensors, drawn in that order from one generator."""
    g = torch.Generator().manual_seed(seed)
    x = make_x(M, d, g, outliers)
    w_gate, w_up, w_down = make_weights(d, F, g)
    return x, w_gate, w_up, w_down


def make_config_inputs(name: str, seed: int = 0, max_rows: int | None = None):
    """Inputs of a named configuration.  `max_rows` keeps only the first rows of x (rows are
    independent); the full x is still drawn so that the weights do not depend on max_rows."""
    cfg = CONFIGS[name]
    g = torch.Generator().manual_seed(seed)
    if cfg.ragged:
        # lengths first, then x (with outliers), then the weights, all from one generator
        lengths = torch.randint(1, 2048 + 1, (32,), generator=g)
        M = int(lengths.sum())
    else:
        M = cfg.M
    x = make_x(M, cfg.d, g, outliers=cfg.ragged)
    if max_rows is not None:
        x = x[:max_rows].contiguous()
    w_gate, w_up, w_down = make_weights(cfg.d, cfg.F, g)
    return x, w_gate, w_up, w_down


def kaiming_uniform_bf16(rows: int, cols: int, g: torch.Generator) -> torch.Tensor:
    """U(-1/sqrt(cols), 1/sqrt(cols)) in bf16: what init.kaiming_uniform_(w, a=sqrt(5)) gives, the
    distribution the reference's numeric_tests.py:8-10,35-38 uses for both operands."""
    bound = 1.0 / (cols ** 0.5)
    return ((torch.rand((rows, cols), generator=g, dtype=torch.float32) * 2.0 - 1.0) * bound).to(torch.bfloat16)
