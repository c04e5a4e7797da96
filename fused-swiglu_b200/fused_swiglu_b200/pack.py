"""Weight layouts on either side of the kernels.

The reference op takes one packed matrix W1W3 [2F, d] whose even rows are the up (linear)
projection and whose odd rows are the gate (SiLU) projection (csrc/SwiGLU/swiglu.cu:376-383,
numeric_tests.py:41-43).  Model checkpoints carry separate gate_proj / up_proj / down_proj
matrices.  These helpers convert between the two and cut Megatron-style tensor-parallel
shards: W_gate / W_up split by rows of F (column-parallel), W_down split along its F axis
(row-parallel), so every rank produces a full-shape partial output to be summed.
"""
from __future__ import annotations

import torch


def interleave_up_gate(W_up: torch.Tensor, W_gate: torch.Tensor) -> torch.Tensor:
    """[F, d] x 2 -> W1W3 [2F, d] with row 2j = up_j, row 2j+1 = gate_j."""
    if W_up.shape != W_gate.shape:
        raise ValueError("W_up and W_gate must have the same shape")
    F, d = W_up.shape
    out = torch.empty((2 * F, d), dtype=W_up.dtype, device=W_up.device)
    out[0::2] = W_up
    out[1::2] = W_gate
    return out


def split_up_gate(W1W3: torch.Tensor):
    """W1W3 [2F, d] -> (W_up [F, d], W_gate [F, d]), contiguous copies."""
    if W1W3.size(0) % 2 != 0:
        raise ValueError("W1W3 needs an even number of rows")
    return W1W3[0::2].contiguous(), W1W3[1::2].contiguous()


def shard_bounds(F: int, world_size: int, rank: int, align: int = 8):
    """[lo, hi) of rank's slice of the hidden dimension; every slice but the last is a multiple
    of `align` (TMA needs 16-byte row pitches, i.e. 8 bf16)."""
    if not 0 <= rank < world_size:
        raise ValueError("rank out of range")
    per = (F + world_size - 1) // world_size
    per = (per + align - 1) // align * align
    lo = min(rank * per, F)
    hi = min(lo + per, F)
    return lo, hi


def shard_mlp_weights(W_gate: torch.Tensor, W_up: torch.Tensor, W_down: torch.Tensor, world_size: int, rank: int):
    """Rank-local (W_gate[lo:hi], W_up[lo:hi], W_down[:, lo:hi]) as contiguous tensors."""
    F = W_gate.size(0)
    lo, hi = shard_bounds(F, world_size, rank)
    return (W_gate[lo:hi].contiguous(), W_up[lo:hi].contiguous(), W_down[:, lo:hi].contiguous())


def fold_norm_weight(W: torch.Tensor, gamma: torch.Tensor) -> torch.Tensor:
    """W [F, d] with the RMSNorm weight vector gamma [d] multiplied into its columns (fp32 product,
    one rounding back to W's dtype): (x * s * gamma) W^T == s * (x (W * gamma)^T), so the norm in front
    of the MLP costs one statistic per row (ops.rms_scale) and nothing else at run time."""
    if gamma.dim() != 1 or gamma.numel() != W.size(1):
        raise ValueError("gamma must have one entry per input feature")
    return (W.float() * gamma.float().to(W.device)[None, :]).to(W.dtype)
