"""GPU parity tests: every compute call goes through the C ABI (ctypes) and is compared with
the CPU oracle on the same seeded inputs, with the committed golden fixtures, and - at the
full benchmark sizes - through row-subset oracles and size-independent properties.

Tolerances (bf16 tensors, fp32 accumulation), written out per test:
  * against the oracle with the SAME rounding points (fp32 acc, fp32 gate, one bf16 rounding):
    at most one bf16 ulp on entries where the fp32 value sits next to a rounding boundary;
    gated on rel-Fro <= 1e-3 and scaled max-abs <= 2^-7;
  * against the fp32 expression (silu(x Wg^T) * (x Wu^T)) Wd^T: rel-Fro <= 5e-3 everywhere;
    raw max-abs <= 2e-2 where |out| stays below 8 (configuration 1), scaled max-abs
    (max-abs / max|ref|) <= 8e-3 elsewhere, because half a bf16 ulp of the largest outputs
    already exceeds 2e-2 there.
"""
import os

import numpy as np
import pytest
import torch

from oracle import swiglu_oracle as orc

pytestmark = pytest.mark.gpu

REL_FRO_SAME_ROUNDING = 1e-3
REL_FRO_GRADED = 5e-3
MAX_ABS_GRADED = 2e-2
SCALED_MAX_ABS = 8e-3


def f32(t):
    return t.detach().float().cpu().numpy()


def bf16_from_bits(a, dev):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16).to(dev)


@pytest.fixture(scope="module")
def fsw(cuda_dev):
    import fused_swiglu_b200 as pkg

    yield pkg
    torch.cuda.synchronize()
    assert pkg.capi.device_status() == 0, "device watchdog tripped during the module"


def healthy(fsw):
    torch.cuda.synchronize()
    assert fsw.capi.device_status() == 0


# ------------------------------------------------------------------ golden fixtures
@pytest.mark.parametrize("name", ["gateup_interleaved_small.npz", "gateup_interleaved_unit.npz"])
def test_packed_op_against_golden(fsw, cuda_dev, golden_dir, name):
    z = np.load(os.path.join(golden_dir, name))
    A, B = bf16_from_bits(z["A"], cuda_dev), bf16_from_bits(z["B"], cuda_dev)
    out = fsw.ops.fused_swiglu_bf16(A, B)
    healthy(fsw)
    assert out.shape == (A.size(0), B.size(0) // 2) and out.dtype == torch.bfloat16
    m = orc.error_metrics(f32(out), z["out_fp32"])
    # fp32 reference lines vs one bf16 rounding of the result: half an ulp, 2^-9 relative
    assert m["rel_fro"] <= 3e-3, m
    # and the reference's own bf16-eager oracle differs from us by its extra roundings only
    m2 = orc.error_metrics(f32(out), orc.bf16_bits_to_f32(z["out_eager_bf16"]))
    assert m2["rel_fro"] <= REL_FRO_GRADED, m2
    # same rounding points -> (almost) bit-exact
    same = orc.gateup_interleaved_fp32acc(orc.bf16_bits_to_f32(z["A"]), orc.bf16_bits_to_f32(z["B"]))
    m3 = orc.error_metrics(f32(out), same)
    assert m3["rel_fro"] <= REL_FRO_SAME_ROUNDING and m3["scaled_max_abs"] <= 2.0 ** -7, m3
    assert (f32(out) != same).mean() < 0.02


@pytest.mark.parametrize("name", ["mlp_small.npz", "mlp_ragged_outliers.npz"])
def test_mlp_against_golden(fsw, cuda_dev, golden_dir, name):
    z = np.load(os.path.join(golden_dir, name))
    x, wg, wu, wd = (bf16_from_bits(z[k], cuda_dev) for k in ("x", "w_gate", "w_up", "w_down"))
    out = fsw.ops.fused_swiglu_mlp_bf16(x, wg, wu, wd)
    healthy(fsw)
    m = orc.error_metrics(f32(out), z["out_fp32"])
    assert m["rel_fro"] <= REL_FRO_GRADED and m["scaled_max_abs"] <= SCALED_MAX_ABS, m


# ------------------------------------------------------------------ oracle, same rounding points
SHAPES = [
    (1, 64, 8), (1, 8, 8), (5, 72, 40), (127, 64, 128), (128, 64, 128), (129, 192, 136), (200, 520, 264),
    (256, 4096, 256), (300, 1000, 520), (1024, 512, 1152),
]


@pytest.mark.parametrize("M,d,F", SHAPES)
def test_gateup_split_matches_oracle(fsw, cuda_dev, M, d, F):
    x, wg, wu, _ = fsw.inputs.make_mlp_inputs(M, d, F, seed=M + d + F)
    wg, wu = wg * 25, wu * 25  # unit-scale pre-activations so that SiLU is exercised off its linear part
    h = fsw.ops.fused_swiglu_gateup_bf16(x.to(cuda_dev), wg.to(cuda_dev), wu.to(cuda_dev))
    healthy(fsw)
    ref = orc.gateup_split_fp32acc(f32(x), f32(wg), f32(wu))
    m = orc.error_metrics(f32(h), ref)
    assert m["rel_fro"] <= REL_FRO_SAME_ROUNDING and m["scaled_max_abs"] <= 2.0 ** -7, m


@pytest.mark.parametrize("M,d,F", SHAPES)
def test_packed_and_split_ops_agree_bitwise(fsw, cuda_dev, M, d, F):
    x, wg, wu, _ = fsw.inputs.make_mlp_inputs(M, d, F, seed=1)
    x, wg, wu = x.to(cuda_dev), (wg * 25).to(cuda_dev), (wu * 25).to(cuda_dev)
    a = fsw.ops.fused_swiglu_gateup_bf16(x, wg, wu)
    b = fsw.ops.fused_swiglu_bf16(x, fsw.pack.interleave_up_gate(wu, wg))
    healthy(fsw)
    assert torch.equal(a, b)


@pytest.mark.parametrize("M,d,F", SHAPES)
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_down_matches_oracle(fsw, cuda_dev, M, d, F, out_dtype):
    g = torch.Generator().manual_seed(M * 7 + F)
    h = torch.randn((M, F), generator=g).to(torch.bfloat16)
    wd = (torch.randn((d, F), generator=g) / F ** 0.5).to(torch.bfloat16)
    out = fsw.ops.swiglu_down_bf16(h.to(cuda_dev), wd.to(cuda_dev), out_dtype=out_dtype)
    healthy(fsw)
    ref = f32(h) @ f32(wd).T
    if out_dtype == torch.bfloat16:
        m = orc.error_metrics(f32(out), orc.bf16_round(ref))
        assert m["rel_fro"] <= REL_FRO_SAME_ROUNDING and m["scaled_max_abs"] <= 2.0 ** -7, m
    else:
        m = orc.error_metrics(f32(out), ref)
        assert m["rel_fro"] <= 1e-5, m


@pytest.mark.parametrize("M,d,F", [(1, 64, 8), (7, 136, 200), (64, 256, 512), (65, 256, 512), (333, 1000, 520)])
def test_mlp_matches_pipeline_oracle(fsw, cuda_dev, M, d, F):
    x, wg, wu, wd = fsw.inputs.make_mlp_inputs(M, d, F, seed=9)
    out = fsw.ops.fused_swiglu_mlp_bf16(x.to(cuda_dev), wg.to(cuda_dev), wu.to(cuda_dev), wd.to(cuda_dev))
    healthy(fsw)
    a = [f32(t) for t in (x, wg, wu, wd)]
    m = orc.error_metrics(f32(out), orc.mlp_bf16_pipeline(*a))
    assert m["rel_fro"] <= REL_FRO_SAME_ROUNDING, m
    m2 = orc.error_metrics(f32(out), orc.mlp_fp32(*a))
    assert m2["rel_fro"] <= REL_FRO_GRADED and m2["scaled_max_abs"] <= SCALED_MAX_ABS, m2


@pytest.mark.parametrize("M,d,F", [(16, 4096, 14336), (33, 4096, 14336), (64, 4096, 14336), (64, 128, 16384),
                                   (40, 520, 4104)])
def test_small_batch_reduction_paths_agree_bitwise(fsw, cuda_dev, M, d, F):
    """The small-batch kernel combines the k-ranges of a row-block of W_down either from the workspace or from
    copies of the partial tiles in shared memory (bulk copies into the idle rings; what does not fit stays in
    the workspace).  Same values, same order: the outputs must be identical, with and without a residual and
    in both output types; (64, 128, 16384) has more ranges per row-block than shared memory holds."""
    x, wg, wu, wd = fsw.inputs.make_mlp_inputs(M, d, F, seed=21)
    args = [t.to(cuda_dev) for t in (x, wg, wu, wd)]
    res = torch.randn((M, d), generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).to(cuda_dev)
    outs = {}
    for mode in ("0", "1"):
        old = os.environ.get("FSWIGLU_DECODE_SMEMRED")
        os.environ["FSWIGLU_DECODE_SMEMRED"] = mode
        try:
            outs[mode] = (fsw.ops.fused_swiglu_mlp_bf16(*args), fsw.ops.fused_swiglu_mlp_bf16(*args, residual=res),
                          fsw.ops.fused_swiglu_mlp_bf16(*args, out_dtype=torch.float32))
            healthy(fsw)
        finally:
            if old is None:
                os.environ.pop("FSWIGLU_DECODE_SMEMRED", None)
            else:
                os.environ["FSWIGLU_DECODE_SMEMRED"] = old
    for a, b in zip(outs["0"], outs["1"]):
        assert torch.equal(a, b)
    default = fsw.ops.fused_swiglu_mlp_bf16(*args)
    assert torch.equal(default, outs["0"][0])
    m = orc.error_metrics(f32(default), orc.mlp_fp32(*[f32(t) for t in (x, wg, wu, wd)]))
    assert m["rel_fro"] <= REL_FRO_GRADED and m["scaled_max_abs"] <= SCALED_MAX_ABS, m


def test_very_tall_problems_run_as_row_slabs_with_identical_results(fsw, cuda_dev):
    """Above 12288 rows the tiled GEMMs are launched slab by slab (about 8192 rows each); rows are independent,
    so the result must equal the single-launch result bit for bit, with every option."""
    M, d, F = 20011, 256, 520
    x, wg, wu, wd = (t.to(cuda_dev) for t in fsw.inputs.make_mlp_inputs(M, d, F, seed=17))
    scale = (0.5 + torch.rand((M,), generator=torch.Generator().manual_seed(3))).to(cuda_dev)
    res = torch.randn((M, d), generator=torch.Generator().manual_seed(4)).to(torch.bfloat16).to(cuda_dev)
    outs = {}
    for mode in ("0", None):
        old = os.environ.get("FSWIGLU_TALL_SLAB")
        if mode is None:
            os.environ.pop("FSWIGLU_TALL_SLAB", None)
        else:
            os.environ["FSWIGLU_TALL_SLAB"] = mode
        try:
            before = fsw.capi.launch_count()
            plain = fsw.ops.fused_swiglu_mlp_bf16(x, wg, wu, wd)
            launches = fsw.capi.launch_count() - before
            outs[mode] = (plain, fsw.ops.fused_swiglu_mlp_bf16(x, wg, wu, wd, residual=res, row_scale=scale),
                          fsw.ops.fused_swiglu_mlp_bf16(x, wg, wu, wd, out_dtype=torch.float32), launches)
            healthy(fsw)
        finally:
            if old is None:
                os.environ.pop("FSWIGLU_TALL_SLAB", None)
            else:
                os.environ["FSWIGLU_TALL_SLAB"] = old
    assert outs["0"][3] == 2 and outs[None][3] == 6  # one launch per GEMM; three slabs per GEMM
    for a, b in zip(outs["0"][:3], outs[None][:3]):
        assert torch.equal(a, b)
    rows = [0, 7167, 7168, 14335, 14336, 20010]  # the slab edges (slabs of 7168, 7168 and 5675 rows)
    m = orc.error_metrics(f32(outs[None][0][rows]), orc.mlp_fp32(*[f32(t) for t in (x[rows], wg, wu, wd)]))
    assert m["rel_fro"] <= REL_FRO_GRADED and m["scaled_max_abs"] <= SCALED_MAX_ABS, m


# ------------------------------------------------------------------ the benchmark configurations
def test_config1_full_size_within_published_tolerance(fsw, cuda_dev):
    """Configuration 1 (M=512, d=1024, F=2816): whole output vs the fp32 expression,
    max-abs <= 2e-2 and rel-Fro <= 5e-3."""
    x, wg, wu, wd = fsw.inputs.make_config_inputs("c1_cpu_small")
    out = fsw.ops.fused_swiglu_mlp_bf16(x.to(cuda_dev), wg.to(cuda_dev), wu.to(cuda_dev), wd.to(cuda_dev))
    healthy(fsw)
    m = orc.error_metrics(f32(out), orc.mlp_fp32(*[f32(t) for t in (x, wg, wu, wd)]))
    assert m["max_abs"] <= MAX_ABS_GRADED and m["rel_fro"] <= REL_FRO_GRADED, m


def _rows_to_check(M, n=96, seed=0):
    rng = np.random.default_rng(seed)
    edge = [r for r in (0, 1, 127, 128, 129, 255, 256, M - 129, M - 128, M - 2, M - 1) if 0 <= r < M]
    rand = rng.choice(M, size=min(n, M), replace=False).tolist()
    return sorted(set(edge + rand))


@pytest.mark.parametrize("name", ["c2_llama2_7b_prefill", "c3_llama3_8b_decode_m1", "c3_llama3_8b_decode_m4",
                                  "c3_llama3_8b_decode_m16", "c3_llama3_8b_decode_m64"])
def test_full_size_configs_row_subset(fsw, cuda_dev, name):
    """Full-size single-GPU configurations: the GPU runs all M rows; tile-edge rows and a random
    sample of rows (all columns) are checked against the fp32 expression on the CPU."""
    x, wg, wu, wd = fsw.inputs.make_config_inputs(name)
    xd, wgd, wud, wdd = (t.to(cuda_dev) for t in (x, wg, wu, wd))
    out = fsw.ops.fused_swiglu_mlp_bf16(xd, wgd, wud, wdd)
    healthy(fsw)
    rows = _rows_to_check(x.size(0))
    ref = orc.mlp_fp32(f32(x[rows]), f32(wg), f32(wu), f32(wd))
    m = orc.error_metrics(f32(out[rows]), ref)
    assert m["rel_fro"] <= REL_FRO_GRADED and m["scaled_max_abs"] <= SCALED_MAX_ABS, m
    # size-independent properties on the full output
    out2 = fsw.ops.fused_swiglu_mlp_bf16(xd, wgd, wud, wdd)
    assert torch.equal(out, out2), "not deterministic"
    if x.size(0) >= 256:
        # A row's result must not depend on where the row sits in the batch.  Bit for bit when every tile
        # is reduced in one piece; with the split last wave (default) a row that lands in one of the shared
        # tiles is summed in a different order, so there the comparison is within the same-rounding tolerance.
        perm = torch.randperm(x.size(0), generator=torch.Generator().manual_seed(1)).to(cuda_dev)
        xp = xd[perm].contiguous()
        out_p = fsw.ops.fused_swiglu_mlp_bf16(xp, wgd, wud, wdd)
        m = orc.error_metrics(f32(out_p), f32(out[perm]))
        assert m["rel_fro"] <= REL_FRO_SAME_ROUNDING and m["scaled_max_abs"] <= 2.0 ** -7, m
        os.environ["FSWIGLU_TAIL_SPLITK"] = "0"
        try:
            a = fsw.ops.fused_swiglu_mlp_bf16(xd, wgd, wud, wdd)
            b = fsw.ops.fused_swiglu_mlp_bf16(xp, wgd, wud, wdd)
        finally:
            del os.environ["FSWIGLU_TAIL_SPLITK"]
        assert torch.equal(b, a[perm]), "rows are not independent of their position"
    out_neg = fsw.ops.fused_swiglu_mlp_bf16(xd, wgd, wud, (-wdd).contiguous())
    assert torch.equal(out_neg, -out), "not odd in W_down"
    out_scaled = fsw.ops.fused_swiglu_mlp_bf16(xd, wgd, wud, (wdd * 2).contiguous())
    assert torch.equal(out_scaled, out * 2), "power-of-two scaling of W_down is not exact"
    healthy(fsw)


@pytest.mark.parametrize("name,world", [("c4_llama3_70b_prefill", 8), ("c5_ragged_13b", 8)])
def test_tp_shard_partials_sum_to_oracle(fsw, cuda_dev, name, world):
    """The tensor-parallel configurations on ONE GPU: every rank's shard is run in turn, the fp32
    partial sums are added in fp32 and rounded once, exactly what the collective does; a row sample
    is compared with the fp32 expression.  Covers F/8 = 1728 (not a multiple of 128) and ragged M."""
    max_rows = 640 if name.startswith("c4") else 414  # 414 = 3*128 + 30: same remainder as M = 32414
    x, wg, wu, wd = fsw.inputs.make_config_inputs(name, max_rows=max_rows)
    xd = x.to(cuda_dev)
    acc = torch.zeros((x.size(0), wd.size(0)), dtype=torch.float32, device=cuda_dev)
    for r in range(world):
        g, u, dn = fsw.pack.shard_mlp_weights(wg, wu, wd, world, r)
        acc += fsw.ops.fused_swiglu_mlp_bf16(xd, g.to(cuda_dev), u.to(cuda_dev), dn.to(cuda_dev),
                                             out_dtype=torch.float32)
    healthy(fsw)
    out = torch.empty_like(acc, dtype=torch.bfloat16)
    import ctypes
    rc = fsw.capi.lib.fswiglu_cast_f32_to_bf16(ctypes.c_void_p(acc.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                                                acc.numel(), None)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(out, acc.to(torch.bfloat16)), "cast kernel differs from round-to-nearest-even"
    rows = _rows_to_check(x.size(0), n=64)
    ref = orc.mlp_fp32(f32(x[rows]), f32(wg), f32(wu), f32(wd))
    m = orc.error_metrics(f32(out[rows]), ref)
    assert m["rel_fro"] <= REL_FRO_GRADED and m["scaled_max_abs"] <= SCALED_MAX_ABS, m


# ------------------------------------------------------------------ edges and the boundary
def test_empty_batch_is_a_no_op(fsw, cuda_dev):
    x = torch.empty((0, 64), dtype=torch.bfloat16, device=cuda_dev)
    w = torch.zeros((16, 64), dtype=torch.bfloat16, device=cuda_dev)
    assert fsw.ops.fused_swiglu_gateup_bf16(x, w, w).shape == (0, 16)
    assert fsw.ops.fused_swiglu_mlp_bf16(x, w, w, w.t().contiguous()).shape == (0, 64)
    healthy(fsw)


def test_outputs_do_not_write_outside_their_rows_and_columns(fsw, cuda_dev):
    """Canary-padded outputs (no sanitizer on this pool): strided output views inside a buffer filled
    with a sentinel; everything outside the view must be untouched."""
    M, d, F = 200, 136, 264
    x, wg, wu, wd = fsw.inputs.make_mlp_inputs(M, d, F, seed=4)
    x, wg, wu, wd = (t.to(cuda_dev) for t in (x, wg, wu, wd))
    sentinel = 1234.0
    big = torch.full((M + 16, F + 24), sentinel, dtype=torch.bfloat16, device=cuda_dev)
    view = big[8:8 + M, 8:8 + F]  # row pitch F+24 (16-byte multiple), base 16 bytes into the row
    import ctypes
    rc = fsw.capi.lib.fswiglu_gateup_bf16(ctypes.c_void_p(x.data_ptr()), d, ctypes.c_void_p(wg.data_ptr()), d,
                                          ctypes.c_void_p(wu.data_ptr()), ctypes.c_void_p(view.data_ptr()), F + 24,
                                          M, F, d, 0, None)
    assert rc == 0
    healthy(fsw)
    ref = fsw.ops.fused_swiglu_gateup_bf16(x, wg, wu)
    assert torch.equal(view, ref)
    mask = torch.ones_like(big, dtype=torch.bool)
    mask[8:8 + M, 8:8 + F] = False
    assert bool((big[mask] == sentinel).all())
    # odd pitch / unaligned base: scalar store path
    big2 = torch.full((M + 2, F + 3), sentinel, dtype=torch.bfloat16, device=cuda_dev)
    view2 = big2[1:1 + M, 1:1 + F]
    rc = fsw.capi.lib.fswiglu_gateup_bf16(ctypes.c_void_p(x.data_ptr()), d, ctypes.c_void_p(wg.data_ptr()), d,
                                          ctypes.c_void_p(wu.data_ptr()), ctypes.c_void_p(view2.data_ptr()), F + 3,
                                          M, F, d, 0, None)
    assert rc == 0
    healthy(fsw)
    assert torch.equal(view2, ref)
    mask2 = torch.ones_like(big2, dtype=torch.bool)
    mask2[1:1 + M, 1:1 + F] = False
    assert bool((big2[mask2] == sentinel).all())


def test_strided_inputs(fsw, cuda_dev):
    """Leading dimensions larger than the row length on every TMA-read operand."""
    M, d, F = 150, 128, 136
    x, wg, wu, wd = fsw.inputs.make_mlp_inputs(M, d, F, seed=6)
    xb = torch.zeros((M, d + 64), dtype=torch.bfloat16, device=cuda_dev)
    xb[:, :d] = x.to(cuda_dev)
    wb = torch.zeros((2, F, d + 8), dtype=torch.bfloat16, device=cuda_dev)
    wb[0, :, :d] = wg.to(cuda_dev)
    wb[1, :, :d] = wu.to(cuda_dev)
    h = fsw.ops.fused_swiglu_gateup_bf16(xb[:, :d], wb[0, :, :d], wb[1, :, :d])
    ref = fsw.ops.fused_swiglu_gateup_bf16(x.to(cuda_dev), wg.to(cuda_dev), wu.to(cuda_dev))
    healthy(fsw)
    assert torch.equal(h, ref)


def test_error_statuses(fsw, cuda_dev):
    import ctypes
    lib, capi = fsw.capi.lib, fsw.capi
    buf = torch.zeros(4096, dtype=torch.bfloat16, device=cuda_dev)
    p = ctypes.c_void_p(buf.data_ptr())
    p_odd = ctypes.c_void_p(buf.data_ptr() + 2)
    assert lib.fswiglu_gateup_bf16(None, 8, p, 8, p, p, 8, 1, 8, 8, 0, None) == capi.ERR_BAD_ARG
    assert lib.fswiglu_gateup_bf16(p, 8, p, 8, p, p, 8, -1, 8, 8, 0, None) == capi.ERR_BAD_ARG
    assert lib.fswiglu_gateup_bf16(p, 12, p, 12, p, p, 8, 1, 8, 12, 0, None) == capi.ERR_SHAPE      # d % 8
    assert lib.fswiglu_gateup_bf16(p, 4, p, 8, p, p, 8, 1, 8, 8, 0, None) == capi.ERR_SHAPE         # ld < d
    assert lib.fswiglu_gateup_bf16(p_odd, 8, p, 8, p, p, 8, 1, 8, 8, 0, None) == capi.ERR_ALIGNMENT
    assert lib.fswiglu_gateup_bf16(p, 8, p, 8, p, p, 8, 1, 8, 8, 1, None) == capi.ERR_BAD_ARG       # packed + w_up
    assert lib.fswiglu_down_bf16(p, 8, p, 8, p, 8, 1, 8, 8, 7, None) == capi.ERR_BAD_ARG            # out dtype
    assert lib.fswiglu_mlp_bf16(p, 8, p, p, 8, p, 8, p, 8, 0, 1, 8, 8, None, 0, None) == capi.ERR_WORKSPACE
    with pytest.raises(RuntimeError, match="bfloat16"):
        fsw.ops.fused_swiglu_bf16(buf.float().view(64, 64), buf.view(64, 64))
    healthy(fsw)


def test_raw_op_writes_half_width_rows_into_full_width_buffer(fsw, cuda_dev):
    """bench_swiglu.py:91,106 passes C [M, N] and ldC = N: the [M, N/2] result is written densely at
    row stride N/2 into the first M*N/2 elements, the rest of C stays untouched."""
    M, K, N = 96, 128, 320
    g = torch.Generator().manual_seed(3)
    A = fsw.inputs.kaiming_uniform_bf16(M, K, g).to(cuda_dev)
    B = fsw.inputs.kaiming_uniform_bf16(N, K, g).to(cuda_dev)
    C = torch.full((M, N), 7.0, dtype=torch.bfloat16, device=cuda_dev)
    fsw.ops.swiglu_fwd_bf16(M, N, K, A, K, B, K, C, N)
    healthy(fsw)
    want = fsw.ops.fused_swiglu_bf16(A, B)
    assert torch.equal(C.flatten()[: M * N // 2].view(M, N // 2), want)
    assert bool((C.flatten()[M * N // 2:] == 7.0).all())


@pytest.mark.parametrize("M", [2500, 1030, 4096, 4097, 5000, 8200])
def test_host_buffer_entry_point(fsw, cuda_dev, M):
    """Activations in pinned host memory, row slabs pipelined over copy streams.  2500 / 1030: equal slabs with a
    ragged (1030: six-row, small-batch kernel) last one; from 4096 rows the first and last slab are half as tall,
    4097 and 5000 leave a remainder for the slab before the last; from 8192 rows the middle slabs are 2048 rows tall."""
    d, F = 256, 520
    x, wg, wu, wd = fsw.inputs.make_mlp_inputs(M, d, F, seed=8)
    wg, wu, wd = wg.to(cuda_dev), wu.to(cuda_dev), wd.to(cuda_dev)
    xh = x.pin_memory()
    oh = torch.empty((M, d), dtype=torch.bfloat16).pin_memory()
    ws = fsw.ops.host_workspace(M, d, F, cuda_dev)
    fsw.ops.fused_swiglu_mlp_bf16_host(xh, wg, wu, wd, oh, ws)
    healthy(fsw)
    want = fsw.ops.fused_swiglu_mlp_bf16(x.to(cuda_dev), wg, wu, wd)
    assert torch.equal(oh, want.cpu())


def test_launches_are_counted(fsw, cuda_dev):
    x, wg, wu, wd = (t.to(cuda_dev) for t in fsw.inputs.make_mlp_inputs(256, 128, 256, seed=1))
    before = fsw.capi.launch_count()
    fsw.ops.fused_swiglu_mlp_bf16(x, wg, wu, wd)
    assert fsw.capi.launch_count() - before >= 1
    healthy(fsw)


@pytest.mark.parametrize("world,M,d,F", [(4, 520, 264, 1096), (2, 2048, 2560, 528)])
def test_push_reduction_kernels_on_one_gpu(fsw, cuda_dev, world, M, d, F):
    """The tensor-parallel 'push' kernels with all ranks emulated on ONE device, one after the other
    (no kernel waits for another): every rank's down GEMM scatters its bf16 partial rows into the
    owners' receive buffers, then every owner reduces its rows in fp32 and stores the result into
    all outputs.  Checked against the fp32 expression and for identical outputs on all 'ranks'."""
    import ctypes
    lib, capi = fsw.capi.lib, fsw.capi
    # case 1 is ragged (130 rows per owner, shards of 280/280/280/256 hidden units, one-SM kernel);
    # case 2 is large enough (80 pair tiles) for the two-SM kernel to run the scatter epilogue
    x, wg, wu, wd = fsw.inputs.make_mlp_inputs(M, d, F, seed=12)
    rpo = (M + world - 1) // world
    xd = x.to(cuda_dev)
    recv = [torch.full((world, rpo, d), float("nan"), dtype=torch.bfloat16, device=cuda_dev) for _ in range(world)]
    outs = [torch.full((world * rpo, d), float("nan"), dtype=torch.bfloat16, device=cuda_dev) for _ in range(world)]
    PtrArr = ctypes.c_void_p * world
    recv_ptrs = PtrArr(*[t.data_ptr() for t in recv])
    for r in range(world):
        g, u, dn = (t.to(cuda_dev) for t in fsw.pack.shard_mlp_weights(wg, wu, wd, world, r))
        h = fsw.ops.fused_swiglu_gateup_bf16(xd, g, u)
        rc = lib.fswiglu_down_scatter_bf16(ctypes.c_void_p(h.data_ptr()), h.size(1), ctypes.c_void_p(dn.data_ptr()),
                                           dn.size(1), recv_ptrs, world, r, rpo, M, d, h.size(1), None, 0, None)
        assert rc == capi.OK, capi.status_string(rc)
    torch.cuda.synchronize()
    for o in range(world):
        out_ptrs = PtrArr(*[t.data_ptr() + o * rpo * d * 2 for t in outs])
        rc = lib.fswiglu_reduce_bcast_bf16(ctypes.c_void_p(recv[o].data_ptr()), out_ptrs, world, rpo, d, 16, None)
        assert rc == capi.OK, capi.status_string(rc)
    healthy(fsw)
    for t in outs[1:]:
        assert torch.equal(t[:M], outs[0][:M])
    ref = orc.mlp_fp32(*[f32(t) for t in (x, wg, wu, wd)])
    m = orc.error_metrics(f32(outs[0][:M]), ref)
    # bf16 partials on the wire + fp32 accumulation + one rounding
    assert m["rel_fro"] <= REL_FRO_GRADED and m["scaled_max_abs"] <= SCALED_MAX_ABS, m
    # bad arguments are refused before anything is launched
    assert lib.fswiglu_down_scatter_bf16(None, 8, None, 8, recv_ptrs, 9, 0, 8, 8, 8, 8, None, 0, None) == capi.ERR_BAD_ARG
    assert lib.fswiglu_reduce_bcast_bf16(None, out_ptrs, 4, 0, 8, 0, None) == capi.OK


def test_sm_budget_changes_nothing_but_the_grid(fsw, cuda_dev):
    x, wg, wu, wd = (t.to(cuda_dev) for t in fsw.inputs.make_mlp_inputs(700, 256, 520, seed=13))
    want = fsw.ops.fused_swiglu_mlp_bf16(x, wg, wu, wd)
    prev = fsw.capi.lib.fswiglu_set_max_ctas(100)
    try:
        got = fsw.ops.fused_swiglu_mlp_bf16(x, wg, wu, wd)
    finally:
        fsw.capi.lib.fswiglu_set_max_ctas(prev)
    healthy(fsw)
    assert torch.equal(got, want)
