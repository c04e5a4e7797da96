"""The fusions either side of the MLP: RMSNorm statistic applied to the gate-up accumulators, residual
added to the down projection's accumulator, and the graph-capture hygiene of the operator surface.
Compute goes through the C ABI (ctypes) or, for the dispatcher tests, through torch.ops.ASMLLM.

Tolerances: against an oracle with the same rounding points rel-Fro <= 1e-3 and scaled max-abs <= 2^-7;
against the fp32 expression rel-Fro <= 5e-3 and scaled max-abs <= 8e-3 (bf16 tensors, fp32 accumulation).
"""
import contextlib
import os

import numpy as np
import pytest
import torch

from oracle import swiglu_oracle as orc

pytestmark = pytest.mark.gpu


def f32(t):
    return t.detach().float().cpu().numpy()


@contextlib.contextmanager
def env(**kv):
    old = {k: os.environ.get(k) for k in kv}
    try:
        os.environ.update(kv)
        yield
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v


@pytest.fixture(scope="module")
def fsw(cuda_dev):
    import fused_swiglu_b200 as pkg

    yield pkg
    torch.cuda.synchronize()
    assert pkg.capi.device_status() == 0, "device watchdog tripped during the module"


@pytest.mark.parametrize("M,d", [(1, 64), (7, 136), (300, 520), (4096, 4096)])
def test_rms_scale_matches_oracle(fsw, cuda_dev, M, d):
    g = torch.Generator().manual_seed(M + d)
    x = (torch.randn((M, d), generator=g) * 3).to(torch.bfloat16)
    got = fsw.ops.rms_scale(x.to(cuda_dev), 1e-6)
    want = orc.rms_scale(f32(x), 1e-6)
    assert got.dtype == torch.float32 and got.shape == (M,)
    np.testing.assert_allclose(f32(got), want, rtol=2e-6)
    # strided rows
    xb = torch.zeros((M, d + 8), dtype=torch.bfloat16, device=cuda_dev)
    xb[:, :d] = x.to(cuda_dev)
    assert torch.equal(fsw.ops.rms_scale(xb[:, :d], 1e-6), got)


@pytest.mark.parametrize("pair", ["0", "force"])
@pytest.mark.parametrize("M,d,F", [(5, 72, 40), (129, 192, 136), (300, 520, 264)])
def test_gateup_row_scale_matches_oracle(fsw, cuda_dev, pair, M, d, F):
    x, wg, wu, _ = fsw.inputs.make_mlp_inputs(M, d, F, seed=3)
    x, wg, wu = x * 4, wg * 25, wu * 25
    s = torch.rand((M,), generator=torch.Generator().manual_seed(1)) + 0.25
    with env(FSWIGLU_PAIR=pair):
        h = fsw.ops.fused_swiglu_gateup_bf16(x.to(cuda_dev), wg.to(cuda_dev), wu.to(cuda_dev), row_scale=s.to(cuda_dev))
    torch.cuda.synchronize()
    sg = f32(s)[:, None]
    acc_g, acc_u = f32(x) @ f32(wg).T, f32(x) @ f32(wu).T
    ref = orc.bf16_round(orc.silu(sg * acc_g) * (sg * acc_u))
    m = orc.error_metrics(f32(h), ref)
    assert m["rel_fro"] <= 1e-3 and m["scaled_max_abs"] <= 2.0 ** -7, m


@pytest.mark.parametrize("pair", ["0", "force"])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,d,F", [(5, 72, 40), (129, 192, 136), (300, 520, 264)])
def test_down_residual_matches_oracle(fsw, cuda_dev, pair, out_dtype, M, d, F):
    g = torch.Generator().manual_seed(M * 7 + F)
    h = torch.randn((M, F), generator=g).to(torch.bfloat16)
    wd = (torch.randn((d, F), generator=g) / F ** 0.5).to(torch.bfloat16)
    res = (torch.randn((M, d), generator=g) * 2).to(torch.bfloat16)
    with env(FSWIGLU_PAIR=pair):
        out = fsw.ops.swiglu_down_bf16(h.to(cuda_dev), wd.to(cuda_dev), out_dtype=out_dtype, residual=res.to(cuda_dev))
    torch.cuda.synchronize()
    ref = f32(h) @ f32(wd).T + f32(res)
    if out_dtype == torch.bfloat16:
        m = orc.error_metrics(f32(out), orc.bf16_round(ref))
        assert m["rel_fro"] <= 1e-3 and m["scaled_max_abs"] <= 2.0 ** -7, m
    else:
        assert orc.error_metrics(f32(out), ref)["rel_fro"] <= 1e-5
    # a strided residual view, and the result written over the residual itself
    big = torch.zeros((M, d + 16), dtype=torch.bfloat16, device=cuda_dev)
    big[:, :d] = res.to(cuda_dev)
    with env(FSWIGLU_PAIR=pair):
        out2 = fsw.ops.swiglu_down_bf16(h.to(cuda_dev), wd.to(cuda_dev), out_dtype=out_dtype, residual=big[:, :d])
        assert torch.equal(out2, out)
        if out_dtype == torch.bfloat16:
            inplace = res.to(cuda_dev)
            fsw.ops.swiglu_down_bf16(h.to(cuda_dev), wd.to(cuda_dev), out=inplace, residual=inplace)
            assert torch.equal(inplace, out)


@pytest.mark.parametrize("M,d,F", [(4, 256, 512), (64, 256, 512), (65, 256, 520), (300, 520, 1096), (2048, 1024, 2816)])
def test_norm_mlp_residual_matches_fp32_expression(fsw, cuda_dev, M, d, F):
    """out = x + MLP(RMSNorm(x)) in two kernels (row statistic, fused MLP) against the fp32 expression, for
    the small-batch kernel (M <= 64) and both tiled kernels."""
    x, wg, wu, wd = fsw.inputs.make_mlp_inputs(M, d, F, seed=11)
    x = x * 2
    gamma = (1.0 + 0.1 * torch.randn((d,), generator=torch.Generator().manual_seed(2))).to(torch.bfloat16)
    wg_f, wu_f = fsw.pack.fold_norm_weight(wg, gamma), fsw.pack.fold_norm_weight(wu, gamma)
    xd = x.to(cuda_dev)
    scale = fsw.ops.rms_scale(xd, 1e-6)
    out = fsw.ops.fused_swiglu_mlp_bf16(xd, wg_f.to(cuda_dev), wu_f.to(cuda_dev), wd.to(cuda_dev), residual=xd,
                                        row_scale=scale)
    torch.cuda.synchronize()
    assert fsw.capi.device_status() == 0
    ref = orc.norm_mlp_residual_fp32(f32(x), f32(gamma), f32(wg), f32(wu), f32(wd), 1e-6, residual=f32(x))
    m = orc.error_metrics(f32(out), ref)
    assert m["rel_fro"] <= 5e-3 and m["scaled_max_abs"] <= 8e-3, m
    # the MLP term alone (residual removed) is held to the same relative bound
    mlp_ref = ref - f32(x)
    out_nores = fsw.ops.fused_swiglu_mlp_bf16(xd, wg_f.to(cuda_dev), wu_f.to(cuda_dev), wd.to(cuda_dev), row_scale=scale)
    m2 = orc.error_metrics(f32(out_nores), mlp_ref)
    assert m2["rel_fro"] <= 5e-3, m2
    # without options the extended entry point is the plain one, bit for bit
    a = fsw.ops.fused_swiglu_mlp_bf16(xd, wg.to(cuda_dev), wu.to(cuda_dev), wd.to(cuda_dev))
    ones = torch.ones((M,), dtype=torch.float32, device=cuda_dev)
    b = fsw.ops.fused_swiglu_mlp_bf16(xd, wg.to(cuda_dev), wu.to(cuda_dev), wd.to(cuda_dev), row_scale=ones)
    assert torch.equal(a, b)


def test_bad_fusion_arguments_are_refused(fsw, cuda_dev):
    x, wg, wu, wd = (t.to(cuda_dev) for t in fsw.inputs.make_mlp_inputs(16, 64, 128, seed=1))
    with pytest.raises(RuntimeError, match="row_scale"):
        fsw.ops.fused_swiglu_gateup_bf16(x, wg, wu, row_scale=torch.ones((15,), device=cuda_dev))
    with pytest.raises(RuntimeError, match="residual"):
        fsw.ops.fused_swiglu_mlp_bf16(x, wg, wu, wd, residual=x.float())
    import ctypes
    lib, capi = fsw.capi.lib, fsw.capi
    p = ctypes.c_void_p(x.data_ptr())
    odd = ctypes.c_void_p(x.data_ptr() + 2)
    assert lib.fswiglu_down_bf16_ex(p, 8, p, 8, p, 8, 1, 8, 8, 0, odd, 8, None, 0, None) == capi.ERR_ALIGNMENT
    assert lib.fswiglu_down_bf16_ex(p, 8, p, 8, p, 8, 1, 8, 8, 0, p, 4, None, 0, None) == capi.ERR_SHAPE
    assert lib.fswiglu_gateup_bf16_ex(p, 8, p, 8, p, p, 8, 1, 8, 8, 0, None, odd, 1 << 30, None) == capi.ERR_WORKSPACE
    assert lib.fswiglu_rms_scale_f32(p, 8, 1, 8, ctypes.c_float(-1.0), p, None) == capi.ERR_BAD_ARG


# ------------------------------------------------------------------ module and dispatcher
def test_block_module_matches_eager_torch(cuda_dev):
    import fused_mlp_module  # noqa: F401
    from fused_swiglu_b200 import inputs
    from fused_swiglu_b200.module import FusedNormSwiGLUBlock

    hidden, inter = 256, 520
    x, wg, wu, wd = inputs.make_mlp_inputs(6 * 50, hidden, inter, seed=21)
    blk = FusedNormSwiGLUBlock(hidden, inter, eps=1e-5, device=cuda_dev)
    gamma = (1.0 + 0.05 * torch.randn((hidden,), generator=torch.Generator().manual_seed(3))).to(torch.bfloat16)
    with torch.no_grad():
        blk.mlp.gate_proj.copy_(wg)
        blk.mlp.up_proj.copy_(wu)
        blk.mlp.down_proj.copy_(wd)
        blk.norm_weight.copy_(gamma)
    blk.fold()
    got = blk(x.to(cuda_dev).view(6, 50, hidden))
    xf = x.float()
    n = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * gamma.float()
    want = xf + (torch.nn.functional.silu(n @ wg.float().T) * (n @ wu.float().T)) @ wd.float().T
    m = orc.error_metrics(f32(got.reshape(-1, hidden)), want.numpy())
    assert got.shape == (6, 50, hidden) and got.dtype == torch.bfloat16
    assert m["rel_fro"] <= 5e-3 and m["scaled_max_abs"] <= 8e-3, m


def test_ops_survive_graph_capture(cuda_dev):
    """torch.compile(fullgraph=True) of the module and of a function that calls the mutating launcher:
    results equal the eager calls bit for bit, and the write into C is neither dropped nor reordered
    (the op's schema declares it: Tensor(a!) C)."""
    import fused_mlp_module  # noqa: F401
    from fused_swiglu_b200 import inputs, pack
    from fused_swiglu_b200.module import FusedSwiGLUMLP

    x, wg, wu, wd = (t.to(cuda_dev) for t in inputs.make_mlp_inputs(300, 256, 520, seed=5))
    mlp = FusedSwiGLUMLP(256, 520, device=cuda_dev)
    with torch.no_grad():
        mlp.gate_proj.copy_(wg)
        mlp.up_proj.copy_(wu)
        mlp.down_proj.copy_(wd)
    eager = mlp(x)
    compiled = torch.compile(mlp, fullgraph=True, backend="aot_eager")
    assert torch.equal(compiled(x), eager)

    w13 = pack.interleave_up_gate(wu, wg)
    M, K, N = x.size(0), x.size(1), w13.size(0)

    def launch_then_read(A, B, C):
        torch.ops.ASMLLM.swiglu_fwd_bf16_out(M, N, K, A, K, B, K, C, N)
        return C.flatten()[: M * N // 2].view(M, N // 2) * 2

    C1 = torch.zeros((M, N), dtype=torch.bfloat16, device=cuda_dev)
    want = launch_then_read(x, w13, C1)
    C2 = torch.zeros((M, N), dtype=torch.bfloat16, device=cuda_dev)
    got = torch.compile(launch_then_read, fullgraph=True, backend="aot_eager")(x, w13, C2)
    assert torch.equal(got, want) and torch.equal(C1, C2)
    assert bool((C2.flatten()[: M * N // 2] != 0).any()), "the captured graph dropped the write into C"
    out32 = torch.ops.ASMLLM.fused_swiglu_mlp_bf16(x, wg, wu, wd, None, None, True)
    assert out32.dtype == torch.float32
    m = orc.error_metrics(f32(out32.to(torch.bfloat16)), f32(eager))
    assert m["rel_fro"] <= 1e-6, "fp32 output rounded once must equal the bf16 output"
