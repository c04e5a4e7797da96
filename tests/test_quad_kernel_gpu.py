"""The two-SM kernel with 512-row tiles (two accumulators filling TMEM, no second accumulator stage) on
small ragged problems, with several tiles per cluster, and at the 70B size it is chosen for.

FSWIGLU_QUAD=force sends every tiled GEMM through it; FSWIGLU_QUAD=0 / FSWIGLU_PAIR=0 select the 256-row
two-SM kernel / the one-SM kernel for comparison.  The k order and the MMA shape are the same in all three,
so results must agree bit for bit.  Every compute call goes through the C ABI.

Tolerances as in test_parity_gpu.py: same-rounding-points oracle rel-Fro <= 1e-3 and scaled max-abs <= 2^-7;
fp32 expression rel-Fro <= 5e-3 and scaled max-abs <= 8e-3.
"""
import contextlib
import ctypes
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


@contextlib.contextmanager
def sm_budget(fsw, ctas):
    prev = fsw.capi.lib.fswiglu_set_max_ctas(ctas)
    try:
        yield
    finally:
        fsw.capi.lib.fswiglu_set_max_ctas(prev)


@pytest.fixture(scope="module")
def fsw(cuda_dev):
    import fused_swiglu_b200 as pkg

    yield pkg
    torch.cuda.synchronize()
    assert pkg.capi.device_status() == 0, "device watchdog tripped during the module"


def healthy(fsw):
    torch.cuda.synchronize()
    assert fsw.capi.device_status() == 0


def vp(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


QUAD = dict(FSWIGLU_QUAD="force")
ONE_SM = dict(FSWIGLU_QUAD="0", FSWIGLU_PAIR="0")
PAIR = dict(FSWIGLU_QUAD="0", FSWIGLU_PAIR="force", FSWIGLU_TAIL_SPLITK="0")

# (M, d, F, SM budget).  M ragged against the 512-row tile, its 256-row CTA halves and the 128-row sub-tiles;
# F and d not multiples of the tile widths; K below, at and above the ring depth of four 64-wide k-blocks; small
# SM budgets give every cluster several tiles, which is what exercises the accumulator hand-over between tiles.
CASES = [(1, 64, 8, 148), (129, 72, 200, 148), (300, 520, 264, 148), (513, 192, 136, 148), (1100, 256, 712, 4),
         (1100, 1000, 712, 4), (2050, 136, 392, 2), (777, 4104, 264, 6)]


@pytest.mark.parametrize("M,d,F,ctas", CASES)
def test_gated_modes_forced_quad_match_oracle_and_other_kernels(fsw, cuda_dev, M, d, F, ctas):
    x, wg, wu, _ = fsw.inputs.make_mlp_inputs(M, d, F, seed=M + F)
    wg, wu = wg * 25, wu * 25
    xd, gd, ud = x.to(cuda_dev), wg.to(cuda_dev), wu.to(cuda_dev)
    w13 = fsw.pack.interleave_up_gate(ud, gd)
    scale = (0.5 + torch.rand((M,), generator=torch.Generator().manual_seed(1))).to(cuda_dev)
    with env(**QUAD), sm_budget(fsw, ctas):
        before = fsw.capi.launch_count()
        split = fsw.ops.fused_swiglu_gateup_bf16(xd, gd, ud)
        packed = fsw.ops.fused_swiglu_bf16(xd, w13)
        assert fsw.capi.launch_count() - before == 2
        scaled = fsw.ops.fused_swiglu_gateup_bf16(xd, gd, ud, row_scale=scale)
    healthy(fsw)
    with env(**ONE_SM):
        one_sm = fsw.ops.fused_swiglu_gateup_bf16(xd, gd, ud)
        one_sm_scaled = fsw.ops.fused_swiglu_gateup_bf16(xd, gd, ud, row_scale=scale)
    with env(**PAIR), sm_budget(fsw, ctas):
        pair = fsw.ops.fused_swiglu_gateup_bf16(xd, gd, ud)
    healthy(fsw)
    m = orc.error_metrics(f32(split), orc.gateup_split_fp32acc(f32(x), f32(wg), f32(wu)))
    assert m["rel_fro"] <= 1e-3 and m["scaled_max_abs"] <= 2.0 ** -7, m
    assert torch.equal(split, packed), "packed (reference layout) and split weights disagree"
    assert torch.equal(split, one_sm), "512-row and one-SM kernels disagree"
    assert torch.equal(split, pair), "512-row and 256-row two-SM kernels disagree"
    assert torch.equal(scaled, one_sm_scaled)


@pytest.mark.parametrize("M,d,F,ctas", CASES)
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_down_forced_quad_matches_oracle_and_one_sm_kernel(fsw, cuda_dev, M, d, F, ctas, out_dtype):
    g = torch.Generator().manual_seed(M * 3 + F)
    h = torch.randn((M, F), generator=g).to(torch.bfloat16)
    wd = (torch.randn((d, F), generator=g) / F ** 0.5).to(torch.bfloat16)
    res = torch.randn((M, d), generator=g).to(torch.bfloat16).to(cuda_dev)
    hd, wdd = h.to(cuda_dev), wd.to(cuda_dev)
    with env(**QUAD), sm_budget(fsw, ctas):
        out = fsw.ops.swiglu_down_bf16(hd, wdd, out_dtype=out_dtype)
        out_res = fsw.ops.swiglu_down_bf16(hd, wdd, out_dtype=out_dtype, residual=res)
    healthy(fsw)
    with env(**ONE_SM):
        one_sm = fsw.ops.swiglu_down_bf16(hd, wdd, out_dtype=out_dtype)
        one_sm_res = fsw.ops.swiglu_down_bf16(hd, wdd, out_dtype=out_dtype, residual=res)
    healthy(fsw)
    ref = f32(h) @ f32(wd).T
    if out_dtype == torch.bfloat16:
        m = orc.error_metrics(f32(out), orc.bf16_round(ref))
        assert m["rel_fro"] <= 1e-3 and m["scaled_max_abs"] <= 2.0 ** -7, m
    else:
        assert orc.error_metrics(f32(out), ref)["rel_fro"] <= 1e-5
    assert torch.equal(out, one_sm)
    assert torch.equal(out_res, one_sm_res)


def test_forced_quad_strided_and_unaligned_outputs_inside_canaries(fsw, cuda_dev):
    """Output views with a larger pitch (vector stores) and with an odd pitch and base (scalar stores) inside
    sentinel-filled buffers; nothing outside the view may change."""
    M, d, F = 700, 136, 264
    x, wg, wu, _ = (t.to(cuda_dev) for t in fsw.inputs.make_mlp_inputs(M, d, F, seed=4))
    with env(**ONE_SM):
        ref = fsw.ops.fused_swiglu_gateup_bf16(x, wg, wu)
    sentinel = 1234.0
    for pad_r, pad_c, pitch_extra in ((8, 8, 24), (1, 1, 3)):
        big = torch.full((M + 2 * pad_r, F + pitch_extra), sentinel, dtype=torch.bfloat16, device=cuda_dev)
        view = big[pad_r:pad_r + M, pad_c:pad_c + F]
        for interleaved in (0, 1):
            big.fill_(sentinel)
            w0 = fsw.pack.interleave_up_gate(wu, wg) if interleaved else wg
            with env(**QUAD):
                rc = fsw.capi.lib.fswiglu_gateup_bf16(vp(x), d, vp(w0), d, None if interleaved else vp(wu), vp(view),
                                                      F + pitch_extra, M, F, d, interleaved, None)
            assert rc == 0
            healthy(fsw)
            assert torch.equal(view, ref)
            mask = torch.ones_like(big, dtype=torch.bool)
            mask[pad_r:pad_r + M, pad_c:pad_c + F] = False
            assert bool((big[mask] == sentinel).all()), "the kernel wrote outside its output view"


def test_whole_mlp_forced_quad_matches_fp32_expression(fsw, cuda_dev):
    M, d, F = 1300, 520, 1096
    x, wg, wu, wd = fsw.inputs.make_mlp_inputs(M, d, F, seed=3)
    args = [t.to(cuda_dev) for t in (x, wg, wu, wd)]
    with env(**QUAD), sm_budget(fsw, 6):
        out = fsw.ops.fused_swiglu_mlp_bf16(*args)
    with env(**ONE_SM):
        ref_kernel = fsw.ops.fused_swiglu_mlp_bf16(*args)
    healthy(fsw)
    assert torch.equal(out, ref_kernel)
    m = orc.error_metrics(f32(out), orc.mlp_fp32(*[f32(t) for t in (x, wg, wu, wd)]))
    assert m["rel_fro"] <= 5e-3 and m["scaled_max_abs"] <= 8e-3, m


def test_70b_shape_takes_the_512_row_kernel_and_equals_the_256_row_kernel(fsw, cuda_dev):
    """At M = d = 8192, F = 28672 the host picks the 512-row kernel for both GEMMs by itself (49 and 7 waves of
    its tiles); the whole output must equal the 256-row kernel's, bit for bit."""
    x, wg, wu, wd = (t.to(cuda_dev) for t in fsw.inputs.make_config_inputs("c4_llama3_70b_prefill"))
    M, d, F = x.size(0), x.size(1), wg.size(0)
    plan = fsw.capi.lib.fswiglu_plan_kernel
    assert plan(M, F, d, 1) == 2 and plan(M, d, F, 0) == 2
    assert plan(4096, 11008, 4096, 1) == 1 and plan(300, 1096, 520, 1) == 0  # 7B gate-up; a small problem
    with env(FSWIGLU_QUAD="0"):
        assert plan(M, F, d, 1) == 1
    ws = fsw.ops.mlp_workspace(M, d, F, cuda_dev)
    out = fsw.ops.fused_swiglu_mlp_bf16(x, wg, wu, wd, workspace=ws)
    with env(FSWIGLU_QUAD="0"):
        ref = fsw.ops.fused_swiglu_mlp_bf16(x, wg, wu, wd, workspace=ws)
    healthy(fsw)
    assert torch.equal(out, ref)
    with env(FSWIGLU_QUAD="0", FSWIGLU_PAIR="0"):
        assert torch.equal(out, fsw.ops.fused_swiglu_mlp_bf16(x, wg, wu, wd, workspace=ws))
