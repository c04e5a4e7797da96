"""Backward pass of the MLP: the C-ABI entry point and the autograd function against the hand-written
float64 chain rule in the oracle and against PyTorch's own autograd of the eager expression.

Tolerance: every intermediate (g, u, dh, dg, du, h) is rounded to bf16 once and the gradients themselves are
bf16, so each gradient is held to rel-Fro <= 1e-2 against the fp64 oracle on the same bf16 inputs (measured:
about 3e-3 to 5e-3), and the fp32-gradient variant to the same bound (its inputs are the same bf16 intermediates).
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import swiglu_oracle as orc

pytestmark = pytest.mark.gpu

GRAD_REL_FRO = 1e-2


def f32(t):
    return t.detach().float().cpu().numpy()


@pytest.fixture(scope="module")
def fsw(cuda_dev):
    import fused_swiglu_b200 as pkg

    yield pkg
    torch.cuda.synchronize()
    assert pkg.capi.device_status() == 0


@pytest.mark.parametrize("rows,cols", [(1, 8), (7, 72), (64, 64), (300, 520), (1000, 136)])
def test_transpose_pads_with_zeros(fsw, cuda_dev, rows, cols):
    src = torch.randn((rows, cols), generator=torch.Generator().manual_seed(rows)).to(torch.bfloat16).to(cuda_dev)
    dst = fsw.ops.transpose_bf16(src)
    rp = (rows + 7) // 8 * 8
    assert dst.shape == (cols, rp)
    assert torch.equal(dst[:, :rows], src.T)
    assert bool((dst[:, rows:] == 0).all())
    # strided source, destination inside a wider buffer
    big = torch.zeros((rows, cols + 8), dtype=torch.bfloat16, device=cuda_dev)
    big[:, :cols] = src
    wide = torch.full((cols, rp + 16), 7.0, dtype=torch.bfloat16, device=cuda_dev)
    rc = fsw.capi.lib.fswiglu_transpose_bf16(ctypes.c_void_p(big.data_ptr()), cols + 8, ctypes.c_void_p(wide.data_ptr()),
                                             rp + 16, rows, cols, None)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(wide[:, :rp], dst) and bool((wide[:, rp:] == 7.0).all())


@pytest.mark.parametrize("M,N,K", [(5, 40, 72), (300, 264, 520), (520, 1096, 304)])
def test_gemm_tn_matches_fp32(fsw, cuda_dev, M, N, K):
    g = torch.Generator().manual_seed(M + N)
    a = torch.randn((M, K), generator=g).to(torch.bfloat16)
    b = (torch.randn((N, K), generator=g) / K ** 0.5).to(torch.bfloat16)
    c = fsw.ops.gemm_tn_bf16(a.to(cuda_dev), b.to(cuda_dev), out_dtype=torch.float32)
    assert orc.error_metrics(f32(c), f32(a) @ f32(b).T)["rel_fro"] <= 1e-5


@pytest.mark.parametrize("grad_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,d,F", [(8, 64, 128), (37, 136, 200), (300, 520, 1096), (1024, 512, 1408)])
def test_backward_matches_chain_rule_oracle(fsw, cuda_dev, M, d, F, grad_dtype):
    x, wg, wu, wd = fsw.inputs.make_mlp_inputs(M, d, F, seed=M + F)
    wg, wu = wg * 10, wu * 10  # pre-activations of order one, so that the gate's derivative is exercised
    dout = torch.randn((M, d), generator=torch.Generator().manual_seed(7)).to(torch.bfloat16)
    got = fsw.ops.swiglu_mlp_backward(*(t.to(cuda_dev) for t in (x, wg, wu, wd, dout)), grad_dtype=grad_dtype)
    torch.cuda.synchronize()
    assert fsw.capi.device_status() == 0
    want = orc.mlp_backward_fp32(*[f32(t) for t in (x, wg, wu, wd, dout)])
    for name, a, b in zip(("dx", "dW_gate", "dW_up", "dW_down"), got, want):
        assert a.dtype == grad_dtype and tuple(a.shape) == b.shape
        m = orc.error_metrics(f32(a), b)
        assert m["rel_fro"] <= GRAD_REL_FRO, (name, m)
        assert np.isfinite(f32(a)).all()


def test_autograd_function_matches_torch_autograd(fsw, cuda_dev):
    M, d, F = 200, 256, 520
    x, wg, wu, wd = fsw.inputs.make_mlp_inputs(M, d, F, seed=3)
    wg, wu = wg * 10, wu * 10
    leaves = [t.to(cuda_dev).requires_grad_(True) for t in (x, wg, wu, wd)]
    out = fsw.ops.fused_swiglu_mlp(*leaves)
    weight = torch.randn((M, d), generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).to(cuda_dev)
    (out.float() * weight.float()).sum().backward()
    ref_leaves = [t.double().requires_grad_(True) for t in (x, wg, wu, wd)]
    rx, rg, ru, rd = ref_leaves
    ref = (torch.nn.functional.silu(rx @ rg.T) * (rx @ ru.T)) @ rd.T
    (ref * weight.cpu().double()).sum().backward()
    for a, b in zip(leaves, ref_leaves):
        m = orc.error_metrics(f32(a.grad), b.grad.float().numpy())
        assert m["rel_fro"] <= GRAD_REL_FRO, m
    m = orc.error_metrics(f32(out), ref.detach().float().numpy())
    assert m["rel_fro"] <= 5e-3, m


def test_backward_argument_checks(fsw, cuda_dev):
    lib, capi = fsw.capi.lib, fsw.capi
    assert lib.fswiglu_backward_workspace_bytes(0, 8, 8) == 0
    assert lib.fswiglu_backward_workspace_bytes(64, 64, 128) > 3 * 64 * 128 * 2
    buf = torch.zeros(4096, dtype=torch.bfloat16, device=cuda_dev)
    p = ctypes.c_void_p(buf.data_ptr())
    args = (p, 8, p, p, 8, p, 8, p, 8, p, 8, p, p, 8, p, 8)
    assert lib.fswiglu_mlp_backward_bf16(*args, 0, 8, 8, 8, None, 0, None) == capi.ERR_WORKSPACE
    assert lib.fswiglu_mlp_backward_bf16(*args, 5, 8, 8, 8, p, 1 << 20, None) == capi.ERR_BAD_ARG
    assert lib.fswiglu_mlp_backward_bf16(*args, 0, 0, 8, 8, None, 0, None) == capi.OK  # no tokens
