"""nn.Module wrapper around the whole-MLP op, with the parameter names model checkpoints use.

The reference only gestures at a module (bench_swiglu.py:22-32 builds a `Swiglu` module around its
packed op and wraps it in torch.compile, :97); this is the caller's side of the operator boundary:
gate_proj / up_proj / down_proj weights as parameters, any leading batch dimensions, inference only
(the ops are forward-only, like the reference's).  The forward goes through the dispatcher op
`ASMLLM::fused_swiglu_mlp_bf16`, which has CUDA and Meta (shape-only) implementations.
"""
from __future__ import annotations

import torch
from torch import nn


def _load_ops():
    import fused_mlp_module  # noqa: F401  (registers torch.ops.ASMLLM.*)

    return torch.ops.ASMLLM


class FusedSwiGLUMLP(nn.Module):
    """out = down_proj(silu(gate_proj(x)) * up_proj(x)), bias-free, bf16 weights.

    gate_proj.weight / up_proj.weight are [intermediate, hidden], down_proj.weight is
    [hidden, intermediate]: the layout of Llama-family checkpoints, used as is (no packing pass).
    """

    def __init__(self, hidden_size: int, intermediate_size: int, device=None):
        super().__init__()
        if hidden_size % 8 or intermediate_size % 8:
            raise ValueError("hidden_size and intermediate_size must be multiples of 8")
        kw = dict(dtype=torch.bfloat16, device=device)
        self.gate_proj = nn.Parameter(torch.empty((intermediate_size, hidden_size), **kw), requires_grad=False)
        self.up_proj = nn.Parameter(torch.empty((intermediate_size, hidden_size), **kw), requires_grad=False)
        self.down_proj = nn.Parameter(torch.empty((hidden_size, intermediate_size), **kw), requires_grad=False)
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size

    @classmethod
    def from_linears(cls, gate_proj: nn.Linear, up_proj: nn.Linear, down_proj: nn.Linear) -> "FusedSwiGLUMLP":
        """Take over the weights of three bias-free nn.Linear layers (cast to bf16, made contiguous)."""
        for lin in (gate_proj, up_proj, down_proj):
            if lin.bias is not None:
                raise ValueError("the fused MLP has no bias terms")
        mod = cls(gate_proj.in_features, gate_proj.out_features, device=gate_proj.weight.device)
        with torch.no_grad():
            mod.gate_proj.copy_(gate_proj.weight)
            mod.up_proj.copy_(up_proj.weight)
            mod.down_proj.copy_(down_proj.weight)
        return mod

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.size(-1) != self.hidden_size:
            raise RuntimeError(f"expected last dimension {self.hidden_size}, got {x.size(-1)}")
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.hidden_size)
        if x2.dtype != torch.bfloat16:
            x2 = x2.to(torch.bfloat16)
        out = _load_ops().fused_swiglu_mlp_bf16(x2.contiguous(), self.gate_proj, self.up_proj, self.down_proj)
        return out.reshape(*lead, self.hidden_size)


class FusedNormSwiGLUBlock(nn.Module):
    """out = x + down_proj(silu(gate_proj(n)) * up_proj(n)),  n = RMSNorm(x) = x * rsqrt(mean(x^2) + eps) * weight.

    The pre-norm MLP half of a Llama-family block in two kernels instead of six: a one-pass row statistic
    (`rms_scale`) and the fused MLP, which applies the statistic to its fp32 gate / up accumulators and
    adds the residual to the fp32 accumulator of the down projection before the single rounding.  The
    norm's weight vector is multiplied into the columns of gate_proj / up_proj once, by `fold()`; the
    normalised activations are never written to memory.  Inference only, like the ops.
    """

    def __init__(self, hidden_size: int, intermediate_size: int, eps: float = 1e-6, device=None):
        super().__init__()
        self.mlp = FusedSwiGLUMLP(hidden_size, intermediate_size, device=device)
        self.norm_weight = nn.Parameter(torch.ones((hidden_size,), dtype=torch.bfloat16, device=device),
                                        requires_grad=False)
        self.eps = eps
        self._folded = None

    def fold(self) -> None:
        """(Re)compute the gate / up matrices with the norm weight folded in; call after loading weights."""
        from . import pack

        self._folded = (pack.fold_norm_weight(self.mlp.gate_proj.data, self.norm_weight.data),
                        pack.fold_norm_weight(self.mlp.up_proj.data, self.norm_weight.data))

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self._folded is None:
            self.fold()
        ops = _load_ops()
        hidden = self.mlp.hidden_size
        lead = x.shape[:-1]
        x2 = x.reshape(-1, hidden)
        if x2.dtype != torch.bfloat16:
            x2 = x2.to(torch.bfloat16)
        x2 = x2.contiguous()
        scale = ops.rms_scale(x2, self.eps)
        out = ops.fused_swiglu_mlp_bf16(x2, self._folded[0], self._folded[1], self.mlp.down_proj, x2, scale, False)
        return out.reshape(*lead, hidden)
