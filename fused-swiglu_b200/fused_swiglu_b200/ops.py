"""Python mirror of the reference operator surface, on top of the C ABI.

The reference exposes two ops from `fused_mlp_module` (csrc/torch_bindings.cpp:31-36):

    fused_swiglu_bf16(X, W1W3) -> Tensor                       (csrc/SwiGLU/swiglu.cu:538-553)
    swiglu_fwd_bf16(m, n, k, A, ldA, B, ldB, C, ldC) -> None   (csrc/SwiGLU/swiglu.cu:397-525)

Both keep their names, argument order and meaning here (W1W3 packs up rows at even and
gate rows at odd indices; the result is [M, N/2] written at row stride ldC/2), and raise
RuntimeError on a wrong dtype like the reference's TORCH_CHECKs (:475-480).  Added on top:
the split-weight gate-up op, the down projection and the whole-MLP op.

PyTorch is used for device memory and the current stream only; all arithmetic happens
in libfswiglu.so.  Tensors must live on a CUDA device.
"""
from __future__ import annotations

import ctypes

import torch

from . import capi


def _stream_ptr(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _vp(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _require_bf16_cuda(**tensors: torch.Tensor) -> None:
    for name, t in tensors.items():
        if t.dtype != torch.bfloat16:
            raise RuntimeError(f"{name} must be a bfloat16 tensor, got {t.dtype}")
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor (no CPU path exists)")


def _row_major_ld(name: str, t: torch.Tensor) -> int:
    if t.dim() != 2:
        raise RuntimeError(f"{name} must be 2-D, got {t.dim()}-D")
    if t.size(1) > 1 and t.stride(1) != 1:
        raise RuntimeError(f"{name} must have unit stride along its last dimension")
    return t.stride(0) if t.size(0) > 1 else max(t.stride(0), t.size(1))


def swiglu_fwd_bf16(m: int, n: int, k: int, A: torch.Tensor, ldA: int, B: torch.Tensor, ldB: int,
                    C: torch.Tensor, ldC: int) -> None:
    """C[:m, :n/2] (row stride ldC/2) = up * silu(gate) with [up|gate] interleaved rows of B.

    Same contract as the reference launcher: raw leading dimensions in elements, the result
    occupies the first m*n/2 elements of C when ldC == n.
    """
    _require_bf16_cuda(A=A, B=B, C=C)
    if n % 2 != 0 or ldC % 2 != 0:
        raise RuntimeError("n and ldC must be even (up/gate rows are interleaved)")
    with torch.cuda.device(A.device):
        rc = capi.lib.fswiglu_gateup_bf16(_vp(A), ldA, _vp(B), ldB, None, _vp(C), ldC // 2, m, n // 2, k, 1,
                                          ctypes.c_void_p(_stream_ptr(A)))
    capi.check(rc, "swiglu_fwd_bf16")


def fused_swiglu_bf16(X: torch.Tensor, W1W3: torch.Tensor) -> torch.Tensor:
    """out[M, N/2] = (X W1W3^T)[:, 0::2] * silu((X W1W3^T)[:, 1::2]), freshly allocated."""
    _require_bf16_cuda(X=X, W1W3=W1W3)
    M, K = X.size(0), X.size(1)
    N = W1W3.size(0)
    out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=X.device)
    swiglu_fwd_bf16(M, N, K, X, _row_major_ld("X", X), W1W3, _row_major_ld("W1W3", W1W3), out, N)
    return out


def gemm_scratch(device: torch.device | str | int) -> torch.Tensor:
    """Scratch buffer that lets the two-SM kernel split the reduction of its last, partly filled wave
    over all SMs (fswiglu_gemm_scratch_bytes).  Share it only between calls ordered on one stream."""
    return torch.empty(int(capi.lib.fswiglu_gemm_scratch_bytes()), dtype=torch.uint8, device=device)


def _check_row_scale(row_scale: torch.Tensor | None, M: int, device) -> None:
    if row_scale is None:
        return
    if row_scale.dtype != torch.float32 or row_scale.device != device or row_scale.numel() != M or \
            not row_scale.is_contiguous():
        raise RuntimeError("row_scale must be a contiguous float32 tensor of M elements on the device of x")


def _check_residual(residual: torch.Tensor | None, M: int, d: int, device) -> int:
    if residual is None:
        return 0
    if residual.dtype != torch.bfloat16 or residual.device != device or tuple(residual.shape) != (M, d):
        raise RuntimeError("residual must be a bfloat16 tensor [M, d] on the device of x")
    return _row_major_ld("residual", residual)


def rms_scale(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """scale[r] = rsqrt(mean(x[r]^2) + eps) in fp32: the per-row statistic of RMSNorm, for `row_scale`."""
    _require_bf16_cuda(x=x)
    M, d = x.shape
    scale = torch.empty((M,), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        rc = capi.lib.fswiglu_rms_scale_f32(_vp(x), _row_major_ld("x", x), M, d, float(eps), _vp(scale),
                                            ctypes.c_void_p(_stream_ptr(x)))
    capi.check(rc, "rms_scale")
    return scale


def fused_swiglu_gateup_bf16(x: torch.Tensor, W_gate: torch.Tensor, W_up: torch.Tensor,
                             row_scale: torch.Tensor | None = None,
                             scratch: torch.Tensor | None = None) -> torch.Tensor:
    """h[M, F] = silu(s * x W_gate^T) * (s * x W_up^T) with separate (un-interleaved) weights;
    s = optional per-row factor (see rms_scale)."""
    _require_bf16_cuda(x=x, W_gate=W_gate, W_up=W_up)
    _check_row_scale(row_scale, x.size(0), x.device)
    M, d = x.shape
    F = W_gate.size(0)
    if W_up.shape != W_gate.shape or W_gate.size(1) != d:
        raise RuntimeError("W_gate and W_up must both be [F, d]")
    ldw = _row_major_ld("W_gate", W_gate)
    if _row_major_ld("W_up", W_up) != ldw:
        raise RuntimeError("W_gate and W_up must share one leading dimension")
    h = torch.empty((M, F), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        rc = capi.lib.fswiglu_gateup_bf16_ex(_vp(x), _row_major_ld("x", x), _vp(W_gate), ldw, _vp(W_up), _vp(h), F,
                                             M, F, d, 0, _vp(row_scale), _vp(scratch),
                                             0 if scratch is None else scratch.numel(),
                                             ctypes.c_void_p(_stream_ptr(x)))
    capi.check(rc, "fused_swiglu_gateup_bf16")
    return h


def swiglu_down_bf16(h: torch.Tensor, W_down: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
                     out: torch.Tensor | None = None, residual: torch.Tensor | None = None,
                     scratch: torch.Tensor | None = None) -> torch.Tensor:
    """out[M, d] = (residual +) h W_down^T; bf16 result, or fp32 partial sums for tensor-parallel reduction."""
    _require_bf16_cuda(h=h, W_down=W_down)
    M, F = h.shape
    d = W_down.size(0)
    if W_down.size(1) != F:
        raise RuntimeError("W_down must be [d, F]")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise RuntimeError("out_dtype must be bfloat16 or float32")
    if out is None:
        out = torch.empty((M, d), dtype=out_dtype, device=h.device)
    code = capi.OUT_BF16 if out_dtype == torch.bfloat16 else capi.OUT_F32
    ldr = _check_residual(residual, M, d, h.device)
    with torch.cuda.device(h.device):
        rc = capi.lib.fswiglu_down_bf16_ex(_vp(h), _row_major_ld("h", h), _vp(W_down),
                                           _row_major_ld("W_down", W_down), _vp(out), _row_major_ld("out", out), M, d,
                                           F, code, _vp(residual), ldr, _vp(scratch),
                                           0 if scratch is None else scratch.numel(),
                                           ctypes.c_void_p(_stream_ptr(h)))
    capi.check(rc, "swiglu_down_bf16")
    return out


def mlp_workspace(M: int, d: int, F: int, device: torch.device | str | int) -> torch.Tensor:
    """Scratch tensor of the size fswiglu_mlp_bf16 asks for (hidden activations, split-K partials)."""
    nbytes = int(capi.lib.fswiglu_workspace_bytes(M, d, F))
    return torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)


def fused_swiglu_mlp_bf16(x: torch.Tensor, W_gate: torch.Tensor, W_up: torch.Tensor, W_down: torch.Tensor,
                          out_dtype: torch.dtype = torch.bfloat16, workspace: torch.Tensor | None = None,
                          out: torch.Tensor | None = None, residual: torch.Tensor | None = None,
                          row_scale: torch.Tensor | None = None) -> torch.Tensor:
    """out[M, d] = (residual +) (silu(s * x W_gate^T) * (s * x W_up^T)) W_down^T in one C-ABI call;
    s = optional per-row factor (see rms_scale)."""
    _require_bf16_cuda(x=x, W_gate=W_gate, W_up=W_up, W_down=W_down)
    M, d = x.shape
    F = W_gate.size(0)
    if W_up.shape != W_gate.shape or W_gate.size(1) != d or tuple(W_down.shape) != (d, F):
        raise RuntimeError("expected W_gate/W_up [F, d] and W_down [d, F]")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise RuntimeError("out_dtype must be bfloat16 or float32")
    ldw = _row_major_ld("W_gate", W_gate)
    if _row_major_ld("W_up", W_up) != ldw:
        raise RuntimeError("W_gate and W_up must share one leading dimension")
    if out is None:
        out = torch.empty((M, d), dtype=out_dtype, device=x.device)
    if M == 0:
        return out
    if workspace is None:
        workspace = mlp_workspace(M, d, F, x.device)
    code = capi.OUT_BF16 if out_dtype == torch.bfloat16 else capi.OUT_F32
    _check_row_scale(row_scale, M, x.device)
    ldr = _check_residual(residual, M, d, x.device)
    with torch.cuda.device(x.device):
        rc = capi.lib.fswiglu_mlp_bf16_ex(_vp(x), _row_major_ld("x", x), _vp(row_scale), _vp(W_gate), _vp(W_up), ldw,
                                          _vp(W_down), _row_major_ld("W_down", W_down), _vp(residual), ldr,
                                          _vp(out), _row_major_ld("out", out), code, M, d, F, _vp(workspace),
                                          workspace.numel(), ctypes.c_void_p(_stream_ptr(x)))
    capi.check(rc, "fused_swiglu_mlp_bf16")
    return out


def host_workspace(M: int, d: int, F: int, device: torch.device | str | int) -> torch.Tensor:
    nbytes = int(capi.lib.fswiglu_host_workspace_bytes(M, d, F))
    return torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)


def fused_swiglu_mlp_bf16_host(x_host: torch.Tensor, W_gate: torch.Tensor, W_up: torch.Tensor,
                               W_down: torch.Tensor, out_host: torch.Tensor, workspace: torch.Tensor) -> None:
    """Whole MLP with activations in (pinned) host memory; returns once out_host is filled."""
    _require_bf16_cuda(W_gate=W_gate, W_up=W_up, W_down=W_down)
    if x_host.is_cuda or out_host.is_cuda or x_host.dtype != torch.bfloat16 or out_host.dtype != torch.bfloat16:
        raise RuntimeError("x_host and out_host must be bfloat16 host tensors")
    if not (x_host.is_contiguous() and out_host.is_contiguous() and W_gate.is_contiguous()
            and W_up.is_contiguous() and W_down.is_contiguous()):
        raise RuntimeError("host entry point needs contiguous tensors")
    M, d = x_host.shape
    F = W_gate.size(0)
    with torch.cuda.device(W_gate.device):
        rc = capi.lib.fswiglu_mlp_bf16_host(_vp(x_host), _vp(W_gate), _vp(W_up), _vp(W_down), _vp(out_host), M, d, F,
                                            _vp(workspace), workspace.numel(),
                                            ctypes.c_void_p(_stream_ptr(W_gate)))
    capi.check(rc, "fused_swiglu_mlp_bf16_host")


def gemm_tn_bf16(a: torch.Tensor, b: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
                 scratch: torch.Tensor | None = None) -> torch.Tensor:
    """c[M, N] = a[M, K] b[N, K]^T, both operands K-major bf16, fp32 accumulation (the GEMM of the backward pass)."""
    _require_bf16_cuda(a=a, b=b)
    if a.size(1) != b.size(1):
        raise RuntimeError("a and b must share their last dimension")
    return swiglu_down_bf16(a, b, out_dtype=out_dtype, scratch=scratch)


def transpose_bf16(src: torch.Tensor) -> torch.Tensor:
    """[rows, cols] -> [cols, rows rounded up to a multiple of 8], pad columns zero (a K-major GEMM operand)."""
    _require_bf16_cuda(src=src)
    rows, cols = src.shape
    dst = torch.empty((cols, (rows + 7) // 8 * 8), dtype=torch.bfloat16, device=src.device)
    with torch.cuda.device(src.device):
        rc = capi.lib.fswiglu_transpose_bf16(_vp(src), _row_major_ld("src", src), _vp(dst), dst.stride(0), rows, cols,
                                             ctypes.c_void_p(_stream_ptr(src)))
    capi.check(rc, "transpose_bf16")
    return dst


def backward_workspace(M: int, d: int, F: int, device: torch.device | str | int) -> torch.Tensor:
    return torch.empty(max(int(capi.lib.fswiglu_backward_workspace_bytes(M, d, F)), 256), dtype=torch.uint8, device=device)


def swiglu_mlp_backward(x: torch.Tensor, W_gate: torch.Tensor, W_up: torch.Tensor, W_down: torch.Tensor,
                        dout: torch.Tensor, grad_dtype: torch.dtype = torch.bfloat16,
                        workspace: torch.Tensor | None = None):
    """Gradients (dx, dW_gate, dW_up, dW_down) of out = (silu(x Wg^T) * (x Wu^T)) Wd^T for upstream dout [M, d]."""
    _require_bf16_cuda(x=x, W_gate=W_gate, W_up=W_up, W_down=W_down, dout=dout)
    M, d = x.shape
    F = W_gate.size(0)
    if W_up.shape != W_gate.shape or W_gate.size(1) != d or tuple(W_down.shape) != (d, F) or tuple(dout.shape) != (M, d):
        raise RuntimeError("expected W_gate/W_up [F, d], W_down [d, F] and dout [M, d]")
    if grad_dtype not in (torch.bfloat16, torch.float32):
        raise RuntimeError("grad_dtype must be bfloat16 or float32")
    ldw = _row_major_ld("W_gate", W_gate)
    if _row_major_ld("W_up", W_up) != ldw:
        raise RuntimeError("W_gate and W_up must share one leading dimension")
    kw = dict(dtype=grad_dtype, device=x.device)
    dx, dwg, dwu, dwd = (torch.empty((M, d), **kw), torch.empty((F, d), **kw), torch.empty((F, d), **kw),
                         torch.empty((d, F), **kw))
    if M == 0:
        return dx, dwg.zero_(), dwu.zero_(), dwd.zero_()
    if workspace is None:
        workspace = backward_workspace(M, d, F, x.device)
    code = capi.OUT_BF16 if grad_dtype == torch.bfloat16 else capi.OUT_F32
    with torch.cuda.device(x.device):
        rc = capi.lib.fswiglu_mlp_backward_bf16(_vp(x), _row_major_ld("x", x), _vp(W_gate), _vp(W_up), ldw, _vp(W_down),
                                                _row_major_ld("W_down", W_down), _vp(dout), _row_major_ld("dout", dout),
                                                _vp(dx), d, _vp(dwg), _vp(dwu), d, _vp(dwd), F, code, M, d, F,
                                                _vp(workspace), workspace.numel(), ctypes.c_void_p(_stream_ptr(x)))
    capi.check(rc, "swiglu_mlp_backward")
    return dx, dwg, dwu, dwd


class FusedSwiGLUMLPFunction(torch.autograd.Function):
    """Differentiable form of the whole-MLP op: forward = the fused kernels, backward = swiglu_mlp_backward
    (the pre-activations are recomputed there, so only the inputs are kept)."""

    @staticmethod
    def forward(ctx, x, W_gate, W_up, W_down):
        ctx.save_for_backward(x, W_gate, W_up, W_down)
        return fused_swiglu_mlp_bf16(x, W_gate, W_up, W_down)

    @staticmethod
    def backward(ctx, dout):
        x, W_gate, W_up, W_down = ctx.saved_tensors
        dx, dwg, dwu, dwd = swiglu_mlp_backward(x, W_gate, W_up, W_down, dout.contiguous().to(torch.bfloat16))
        return dx, dwg, dwu, dwd


def fused_swiglu_mlp(x: torch.Tensor, W_gate: torch.Tensor, W_up: torch.Tensor, W_down: torch.Tensor) -> torch.Tensor:
    """Whole MLP with autograd support (bf16 CUDA tensors, 2-D x)."""
    return FusedSwiGLUMLPFunction.apply(x, W_gate, W_up, W_down)
