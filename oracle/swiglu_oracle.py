"""CPU oracle for the fused SwiGLU MLP forward path.  TEST INFRASTRUCTURE ONLY.

Nothing that ships may import this module: it is the checker for tests/, for
__graft_entry__.smoke() and for the cpu_baseline / reference legs of bench.py.  The product
path is the CUDA library; it has no CPU fallback.

What is restated here (numpy, fp32 arithmetic, explicit bf16 rounding points):

  * the reference's eager oracle for its packed gate-up op, numeric_tests.py:41-43
        C = A @ B.T ; silu = F.silu(C[:, 1::2]) ; gated = C[:, ::2] * silu
    with bf16 tensors, i.e. every intermediate rounded to bf16  -> gateup_interleaved_eager_bf16
  * the arithmetic of the reference kernel's epilogue, csrc/SwiGLU/swiglu.cu:376-383 and :96
        out = bf16( acc[:, 2c] * silu(acc[:, 2c+1]) ),  acc in fp32, silu(v) = v / (1 + exp(-v))
    -> gateup_interleaved_fp32acc / gateup_split_fp32acc (one rounding, at the end)
  * the whole-MLP expression results are checked against (the benchmark's first configuration):
        out = (silu(x Wg^T) * (x Wu^T)) Wd^T  in fp32                -> mlp_fp32
    and the same with the rounding points of the GPU path (h rounded to bf16 between the
    two GEMMs, result rounded to bf16)                               -> mlp_bf16_pipeline
  * tensor-parallel partial sums (Megatron split over F)             -> mlp_tp_partials

Pinning: the reference ships no golden vectors and no thresholds (numeric_tests.py only prints
statistics), so parity is pinned against outputs of the reference's own eager expression,
executed with PyTorch on CPU in the build container and committed under tests/golden/ (see
tests/golden/make_golden.py); tests/test_oracle.py checks this file against them.
"""
from __future__ import annotations

import numpy as np


# ----------------------------------------------------------------------------------------
# bf16 helpers: bf16 values are carried as float32 arrays whose low 16 mantissa bits are 0.
# ----------------------------------------------------------------------------------------
def bf16_round(a: np.ndarray) -> np.ndarray:
    """Round fp32 to the nearest bf16 (ties to even), return as fp32.  Matches torch's
    .to(torch.bfloat16) and the CUDA cvt.rn.bf16.f32 for finite values and infinities."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    bits = a.view(np.uint32).astype(np.uint64)
    lsb = (bits >> 16) & 1
    rounded = ((bits + 0x7FFF + lsb) >> 16) << 16
    out = (rounded & 0xFFFFFFFF).astype(np.uint32).view(np.float32)
    nan = np.isnan(a)
    if nan.any():
        out = out.copy()
        out[nan] = np.nan
    return out.reshape(a.shape)


def bf16_bits_to_f32(bits_u16: np.ndarray) -> np.ndarray:
    """uint16 bf16 bit patterns -> fp32 values."""
    return (bits_u16.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """fp32 -> uint16 bf16 bit patterns (round to nearest even)."""
    return (bf16_round(a).view(np.uint32) >> 16).astype(np.uint16)


def silu(v: np.ndarray) -> np.ndarray:
    """silu(v) = v / (1 + exp(-v)) in fp32 (csrc/SwiGLU/swiglu.cu:96)."""
    v = np.asarray(v, dtype=np.float32)
    with np.errstate(over="ignore"):
        return (v / (np.float32(1.0) + np.exp(-v))).astype(np.float32)


def _mm(a: np.ndarray, b_t: np.ndarray) -> np.ndarray:
    """a [M,K] times b_t [N,K] transposed, fp32 accumulate."""
    return np.matmul(np.asarray(a, np.float32), np.asarray(b_t, np.float32).T).astype(np.float32)


# ----------------------------------------------------------------------------------------
# packed (interleaved) gate-up op of the reference
# ----------------------------------------------------------------------------------------
def gateup_interleaved_eager_bf16(A: np.ndarray, B: np.ndarray) -> np.ndarray:
    """numeric_tests.py:41-43 on bf16 tensors: GEMM result, SiLU and product each rounded to bf16.
    A [M,K], B [N,K] hold bf16 values (as fp32).  Returns [M, N/2] bf16 values (as fp32)."""
    C = bf16_round(_mm(A, B))                 # C_torch = A @ B.T           (:41)
    s = bf16_round(silu(C[:, 1::2]))          # silu = F.silu(C[:, 1::2])   (:42)
    return bf16_round(C[:, 0::2] * s)         # gated = C[:, ::2] * silu    (:43)


def gateup_interleaved_fp32acc(A: np.ndarray, B: np.ndarray, round_out: bool = True) -> np.ndarray:
    """Kernel semantics (csrc/SwiGLU/swiglu.cu:376-383): fp32 accumulators, even column (up) times
    silu(odd column (gate)) in fp32, one rounding to bf16."""
    C = _mm(A, B)
    out = C[:, 0::2] * silu(C[:, 1::2])
    return bf16_round(out) if round_out else out.astype(np.float32)


def gateup_split_fp32acc(x: np.ndarray, w_gate: np.ndarray, w_up: np.ndarray, round_out: bool = True) -> np.ndarray:
    """h = silu(x Wg^T) * (x Wu^T) with separate weights; same arithmetic as the packed form."""
    out = silu(_mm(x, w_gate)) * _mm(x, w_up)
    return bf16_round(out) if round_out else out.astype(np.float32)


# ----------------------------------------------------------------------------------------
# whole MLP
# ----------------------------------------------------------------------------------------
def mlp_fp32(x: np.ndarray, w_gate: np.ndarray, w_up: np.ndarray, w_down: np.ndarray) -> np.ndarray:
    """(silu(x Wg^T) * (x Wu^T)) Wd^T entirely in fp32: the expression results are held to."""
    h = silu(_mm(x, w_gate)) * _mm(x, w_up)
    return _mm(h, w_down)


def mlp_bf16_pipeline(x, w_gate, w_up, w_down, round_out: bool = True) -> np.ndarray:
    """Rounding points of the GPU path: fp32 acc -> fp32 gate -> bf16 h -> fp32 acc -> bf16 out."""
    h = gateup_split_fp32acc(x, w_gate, w_up, round_out=True)
    out = _mm(h, w_down)
    return bf16_round(out) if round_out else out


def rms_scale(x: np.ndarray, eps: float = 1e-6) -> np.ndarray:
    """Per-row RMSNorm statistic rsqrt(mean(x^2) + eps) in fp32 (float64 accumulation of the mean)."""
    x = np.asarray(x, np.float32)
    ms = (x.astype(np.float64) ** 2).mean(axis=1)
    return (1.0 / np.sqrt(ms + eps)).astype(np.float32)


def norm_mlp_residual_fp32(x, gamma, w_gate, w_up, w_down, eps: float = 1e-6, residual=None) -> np.ndarray:
    """The pre-norm MLP half of a transformer block in fp32:
    out = residual + (silu(n Wg^T) * (n Wu^T)) Wd^T with n = x * rsqrt(mean(x^2) + eps) * gamma.
    The reference has no counterpart (its kernel stops at the gate); this is the expression the fused
    row-scale / residual options of the GPU path are held to."""
    x = np.asarray(x, np.float32)
    n = x * rms_scale(x, eps)[:, None] * np.asarray(gamma, np.float32)[None, :]
    out = mlp_fp32(n, w_gate, w_up, w_down)
    return out if residual is None else out + np.asarray(residual, np.float32)


def mlp_backward_fp32(x, w_gate, w_up, w_down, dout):
    """Gradients of out = (silu(x Wg^T) * (x Wu^T)) Wd^T with respect to x, Wg, Wu, Wd for upstream dout, written
    out by hand in float64 (the chain rule of the expression the forward oracle implements); returned as fp32."""
    x, w_gate, w_up, w_down, dout = (np.asarray(a, np.float64) for a in (x, w_gate, w_up, w_down, dout))
    g, u = x @ w_gate.T, x @ w_up.T
    s = 1.0 / (1.0 + np.exp(-g))
    h = g * s * u
    dh = dout @ w_down
    dg = dh * u * s * (1.0 + g * (1.0 - s))
    du = dh * g * s
    grads = (dg @ w_gate + du @ w_up, dg.T @ x, du.T @ x, dout.T @ h)
    return tuple(a.astype(np.float32) for a in grads)


def mlp_tp_partials(x, w_gate, w_up, w_down, world_size: int, bounds) -> list[np.ndarray]:
    """fp32 partial outputs of a Megatron split over F: rank r uses rows [lo,hi) of W_gate / W_up and
    columns [lo,hi) of W_down, `bounds(F, world_size, r) -> (lo, hi)`.  Their sum is the MLP output."""
    F = w_gate.shape[0]
    parts = []
    for r in range(world_size):
        lo, hi = bounds(F, world_size, r)
        if hi <= lo:
            parts.append(np.zeros((x.shape[0], w_down.shape[0]), np.float32))
            continue
        parts.append(mlp_bf16_pipeline(x, w_gate[lo:hi], w_up[lo:hi], w_down[:, lo:hi], round_out=False))
    return parts


# ----------------------------------------------------------------------------------------
# error metrics (the three numeric_tests.py:49-52 prints, plus max-abs scaled by max|ref|)
# ----------------------------------------------------------------------------------------
def error_metrics(got: np.ndarray, ref: np.ndarray) -> dict:
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    diff = got - ref
    ref_norm = float(np.linalg.norm(ref))
    ref_max = float(np.abs(ref).max()) if ref.size else 0.0
    max_abs = float(np.abs(diff).max()) if diff.size else 0.0
    return {
        "max_abs": max_abs,
        "mean_abs": float(np.abs(diff).mean()) if diff.size else 0.0,
        "rel_fro": float(np.linalg.norm(diff)) / ref_norm if ref_norm > 0 else 0.0,
        "scaled_max_abs": max_abs / ref_max if ref_max > 0 else 0.0,
        "ref_max": ref_max,
    }


def torch_to_f32(t) -> np.ndarray:
    """torch tensor (any float dtype, any device) -> fp32 numpy array."""
    return t.detach().float().cpu().numpy()
