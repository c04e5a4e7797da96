"""The reference's eager PyTorch expressions, runnable on CPU.  TEST INFRASTRUCTURE ONLY.

These are the expressions the reference project checks its kernel against and that this
library's results are held to; nothing that ships may import this file (it is used by tests/, by the fixture
generator tests/golden/make_golden.py and by the cpu_baseline / reference legs of bench.py).

  gateup_interleaved_eager : numeric_tests.py:41-43 (twin: bench_swiglu.py:30-32)
  mlp_eager                : (F.silu(x @ Wg.T) * (x @ Wu.T)) @ Wd.T, the whole-MLP expression
                             of the benchmark's first configuration (the reference itself stops after the gate)
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def gateup_interleaved_eager(A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    C_torch = A @ B.T
    silu = F.silu(C_torch[:, 1::2])
    return C_torch[:, ::2] * silu


def mlp_eager(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    return (F.silu(x @ w_gate.T) * (x @ w_up.T)) @ w_down.T


def mlp_eager_fp32(x, w_gate, w_up, w_down) -> torch.Tensor:
    """Same expression with every operand upcast to fp32 first (bf16 inputs, fp32 arithmetic)."""
    return mlp_eager(x.float(), w_gate.float(), w_up.float(), w_down.float())
