"""The two-SM (cta_group::2) GEMM kernel on small, ragged problems and at the full benchmark sizes.

The host picks the two-SM kernel only for problems of at least one wave of 256-row tiles, so the
small parity shapes elsewhere in this suite never reach it.  Here FSWIGLU_PAIR=force sends every
call through it (and FSWIGLU_PAIR=0 through the one-SM kernel, for bit-level comparison), and
FSWIGLU_TAIL_SPLITK=force makes the split reduction of the last wave happen on small problems too.
Every compute call goes through the C ABI.

Tolerances as in test_parity_gpu.py: same-rounding-points oracle rel-Fro <= 1e-3 and scaled max-abs
<= 2^-7; fp32 expression rel-Fro <= 5e-3 and scaled max-abs <= 8e-3; kernel-vs-kernel comparisons are
bit-exact when the summation order is the same (no split), within the same-rounding tolerance otherwise.
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
        for k, v in kv.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
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


def healthy(fsw):
    torch.cuda.synchronize()
    assert fsw.capi.device_status() == 0


def vp(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


# M in {129, 300, 414}: ragged against the 256-row pair tile and the 128-row halves; F in {200, 264, 1728}:
# not multiples of the 128-column tile; d = 72 / 520 / 1000: K not a multiple of 64.
RAGGED = [(129, 72, 200), (300, 520, 264), (414, 1000, 1728), (1, 64, 8), (256, 512, 128), (513, 192, 136)]


@pytest.mark.parametrize("M,d,F", RAGGED)
def test_gated_modes_forced_pair_match_oracle_and_one_sm_kernel(fsw, cuda_dev, M, d, F):
    x, wg, wu, _ = fsw.inputs.make_mlp_inputs(M, d, F, seed=M + F)
    wg, wu = wg * 25, wu * 25
    xd, gd, ud = x.to(cuda_dev), wg.to(cuda_dev), wu.to(cuda_dev)
    w13 = fsw.pack.interleave_up_gate(ud, gd)
    with env(FSWIGLU_PAIR="force", FSWIGLU_TAIL_SPLITK="0"):
        before = fsw.capi.launch_count()
        split = fsw.ops.fused_swiglu_gateup_bf16(xd, gd, ud)
        packed = fsw.ops.fused_swiglu_bf16(xd, w13)
        assert fsw.capi.launch_count() - before == 2
    with env(FSWIGLU_PAIR="0"):
        one_sm = fsw.ops.fused_swiglu_gateup_bf16(xd, gd, ud)
    healthy(fsw)
    m = orc.error_metrics(f32(split), orc.gateup_split_fp32acc(f32(x), f32(wg), f32(wu)))
    assert m["rel_fro"] <= 1e-3 and m["scaled_max_abs"] <= 2.0 ** -7, m
    assert torch.equal(split, packed), "packed (reference layout) and split weights disagree on the two-SM kernel"
    assert torch.equal(split, one_sm), "two-SM and one-SM kernels disagree"


@pytest.mark.parametrize("M,d,F", RAGGED)
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_down_forced_pair_matches_oracle_and_one_sm_kernel(fsw, cuda_dev, M, d, F, out_dtype):
    g = torch.Generator().manual_seed(M * 3 + F)
    h = torch.randn((M, F), generator=g).to(torch.bfloat16)
    wd = (torch.randn((d, F), generator=g) / F ** 0.5).to(torch.bfloat16)
    hd, wdd = h.to(cuda_dev), wd.to(cuda_dev)
    with env(FSWIGLU_PAIR="force", FSWIGLU_TAIL_SPLITK="0"):
        out = fsw.ops.swiglu_down_bf16(hd, wdd, out_dtype=out_dtype)
    with env(FSWIGLU_PAIR="0"):
        one_sm = fsw.ops.swiglu_down_bf16(hd, wdd, out_dtype=out_dtype)
    healthy(fsw)
    ref = f32(h) @ f32(wd).T
    if out_dtype == torch.bfloat16:
        m = orc.error_metrics(f32(out), orc.bf16_round(ref))
        assert m["rel_fro"] <= 1e-3 and m["scaled_max_abs"] <= 2.0 ** -7, m
    else:
        assert orc.error_metrics(f32(out), ref)["rel_fro"] <= 1e-5
    assert torch.equal(out, one_sm)


def test_forced_pair_strided_and_unaligned_outputs_inside_canaries(fsw, cuda_dev):
    """Output views with a larger pitch (16-byte aligned: vector stores) and with an odd pitch and base
    (scalar stores) inside sentinel-filled buffers; nothing outside the view may change."""
    M, d, F = 300, 136, 264
    x, wg, wu, _ = (t.to(cuda_dev) for t in fsw.inputs.make_mlp_inputs(M, d, F, seed=4))
    with env(FSWIGLU_PAIR="0"):
        ref = fsw.ops.fused_swiglu_gateup_bf16(x, wg, wu)
    sentinel = 1234.0
    for pad_r, pad_c, pitch_extra in ((8, 8, 24), (1, 1, 3)):
        big = torch.full((M + 2 * pad_r, F + pitch_extra), sentinel, dtype=torch.bfloat16, device=cuda_dev)
        view = big[pad_r:pad_r + M, pad_c:pad_c + F]
        for interleaved in (0, 1):
            big.fill_(sentinel)
            w0 = fsw.pack.interleave_up_gate(wu, wg) if interleaved else wg
            with env(FSWIGLU_PAIR="force"):
                rc = fsw.capi.lib.fswiglu_gateup_bf16(vp(x), d, vp(w0), d, None if interleaved else vp(wu), vp(view),
                                                      F + pitch_extra, M, F, d, interleaved, None)
            assert rc == 0
            healthy(fsw)
            assert torch.equal(view, ref)
            mask = torch.ones_like(big, dtype=torch.bool)
            mask[pad_r:pad_r + M, pad_c:pad_c + F] = False
            assert bool((big[mask] == sentinel).all())


@pytest.mark.parametrize("world,M,d,F", [(4, 520, 264, 1096), (3, 300, 520, 264)])
def test_forced_pair_scatter_epilogue(fsw, cuda_dev, world, M, d, F):
    """The reduce-scatter epilogue (rows stored into their owner's receive buffer) on the two-SM kernel,
    ragged sizes, all ranks emulated in turn on one device; compared with the one-SM kernel bit for bit."""
    lib = fsw.capi.lib
    x, wg, wu, wd = fsw.inputs.make_mlp_inputs(M, d, F, seed=12)
    rpo = (M + world - 1) // world
    xd = x.to(cuda_dev)
    PtrArr = ctypes.c_void_p * world
    results = {}
    for mode in ("force", "0"):
        recv = [torch.full((world, rpo, d), float("nan"), dtype=torch.bfloat16, device=cuda_dev) for _ in range(world)]
        ptrs = PtrArr(*[t.data_ptr() for t in recv])
        with env(FSWIGLU_PAIR=mode, FSWIGLU_TAIL_SPLITK="0"):
            for r in range(world):
                g, u, dn = (t.to(cuda_dev) for t in fsw.pack.shard_mlp_weights(wg, wu, wd, world, r))
                h = fsw.ops.fused_swiglu_gateup_bf16(xd, g, u)
                rc = lib.fswiglu_down_scatter_bf16(vp(h), h.size(1), vp(dn), dn.size(1), ptrs, world, r, rpo, M, d,
                                                   h.size(1), None, 0, None)
                assert rc == 0
        healthy(fsw)
        results[mode] = recv
    for owner, (a, b) in enumerate(zip(results["force"], results["0"])):
        rows = min(rpo, M - owner * rpo)
        assert torch.equal(a[:, :rows], b[:, :rows])
    # partial sums of owner 0, summed in fp32 over the source ranks, against the fp32 expression
    acc = results["force"][0].float().sum(dim=0)
    ref = orc.mlp_fp32(*[f32(t) for t in (x[:rpo], wg, wu, wd)])
    m = orc.error_metrics(f32(acc), ref)
    assert m["rel_fro"] <= 5e-3, m


# ------------------------------------------------------------------ split reduction of the last wave
@contextlib.contextmanager
def sm_budget(fsw, ctas):
    prev = fsw.capi.lib.fswiglu_set_max_ctas(ctas)
    try:
        yield
    finally:
        fsw.capi.lib.fswiglu_set_max_ctas(prev)


# (M, d, F, SM budget): the budget makes the tile counts of both stages leave a remainder on the
# clusters (6 and 8 tiles on 5 clusters, 15 and 24 on 7, 54 and 36 on 10, 99 and 144 on 74)
@pytest.mark.parametrize("M,d,F,ctas", [(300, 1024, 264, 10), (513, 2048, 520, 14), (1500, 1536, 1096, 20),
                                        (2304, 4096, 1408, 0)])
def test_split_last_wave_matches_unsplit(fsw, cuda_dev, M, d, F, ctas):
    """FSWIGLU_TAIL_SPLITK=force: the k-blocks of the last wave's tiles are cut into ranges, partial
    accumulators go through the scratch buffer and the last range to arrive finishes each tile.  All three
    modes and both output types against the unsplit kernel (same-rounding tolerance: the summation order
    of the shared tiles differs) and against the oracle; two runs must agree bit for bit (fixed order)."""
    x, wg, wu, wd = fsw.inputs.make_mlp_inputs(M, d, F, seed=M)
    wg, wu = wg * 25, wu * 25
    xd, gd, ud, dd = (t.to(cuda_dev) for t in (x, wg, wu, wd))
    w13 = fsw.pack.interleave_up_gate(ud, gd)
    scratch = fsw.ops.gemm_scratch(cuda_dev)
    scratch.fill_(0xA5)  # the counters are cleared by the call, not by the caller
    with env(FSWIGLU_PAIR="force", FSWIGLU_TAIL_SPLITK="0"), sm_budget(fsw, ctas):
        h0 = fsw.ops.fused_swiglu_gateup_bf16(xd, gd, ud)
        o0 = fsw.ops.swiglu_down_bf16(h0, dd)
        o0f = fsw.ops.swiglu_down_bf16(h0, dd, out_dtype=torch.float32)
    with env(FSWIGLU_PAIR="force", FSWIGLU_TAIL_SPLITK="force"), sm_budget(fsw, ctas):
        h1 = fsw.ops.fused_swiglu_gateup_bf16(xd, gd, ud, scratch=scratch)
        h1b = fsw.ops.fused_swiglu_gateup_bf16(xd, gd, ud, scratch=scratch)
        hp = torch.empty_like(h1)
        rc = fsw.capi.lib.fswiglu_gateup_bf16_ex(vp(xd), d, vp(w13), d, None, vp(hp), F, M, F, d, 1, None, vp(scratch),
                                                 scratch.numel(), None)
        assert rc == 0
        o1 = fsw.ops.swiglu_down_bf16(h0, dd, scratch=scratch)
        o1f = fsw.ops.swiglu_down_bf16(h0, dd, out_dtype=torch.float32, scratch=scratch)
        o1b = fsw.ops.swiglu_down_bf16(h0, dd, scratch=scratch)
    healthy(fsw)
    assert torch.equal(h1, h1b) and torch.equal(o1, o1b), "split reduction is not deterministic"
    assert torch.equal(h1, hp), "packed and split weights disagree under the split reduction"
    for got, want in ((h1, h0), (o1, o0), (o1f, o0f)):
        m = orc.error_metrics(f32(got), f32(want))
        assert m["rel_fro"] <= 1e-3 and m["scaled_max_abs"] <= 2.0 ** -7, m
    m = orc.error_metrics(f32(h1), orc.gateup_split_fp32acc(f32(x), f32(wg), f32(wu)))
    assert m["rel_fro"] <= 1e-3 and m["scaled_max_abs"] <= 2.0 ** -7, m
    m = orc.error_metrics(f32(o1f), f32(h0) @ f32(wd).T)
    assert m["rel_fro"] <= 1e-5, m


@pytest.mark.parametrize("M,d,F,ctas_gu,ctas_dn", [(300, 1024, 264, 10, 14), (513, 2048, 520, 28, 46),
                                                   (1500, 1536, 1096, 100, 60), (4096, 5120, 1408, 0, 0)])
def test_width_split_last_wave_is_bit_identical(fsw, cuda_dev, M, d, F, ctas_gu, ctas_dn):
    """When the last wave's tiles fill at most half of the clusters they are processed as two half-width
    units each (64-row operand boxes, N = 128 MMAs).  Same k order as a whole tile, so every mode and output
    type must equal the unsplit two-SM kernel and the one-SM kernel bit for bit.  The SM budgets make the
    tile counts leave such a remainder: gate-up 6 tiles on 5 clusters, 15 on 14, 54 on 50, 176 on 74; down
    8 on 7, 24 on 23, 36 on 30, 320 on 74."""
    x, wg, wu, wd = fsw.inputs.make_mlp_inputs(M, d, F, seed=M + 1)
    wg, wu = wg * 25, wu * 25
    xd, gd, ud, dd = (t.to(cuda_dev) for t in (x, wg, wu, wd))
    w13 = fsw.pack.interleave_up_gate(ud, gd)
    res = {}
    for name, envs in (("halves", dict(FSWIGLU_PAIR="force", FSWIGLU_TAIL_SPLITK="0")),
                       ("whole", dict(FSWIGLU_PAIR="force", FSWIGLU_TAIL_SPLITK="0", FSWIGLU_TAIL_HALVES="0")),
                       ("one_sm", dict(FSWIGLU_PAIR="0"))):
        with env(**envs), sm_budget(fsw, ctas_gu):
            h = fsw.ops.fused_swiglu_gateup_bf16(xd, gd, ud)
            hp = fsw.ops.fused_swiglu_bf16(xd, w13)
        with env(**envs), sm_budget(fsw, ctas_dn):
            o = fsw.ops.swiglu_down_bf16(h, dd)
            of = fsw.ops.swiglu_down_bf16(h, dd, out_dtype=torch.float32)
        healthy(fsw)
        res[name] = (h, hp, o, of)
    for other in ("whole", "one_sm"):
        for a, b in zip(res["halves"], res[other]):
            assert torch.equal(a, b), other
    m = orc.error_metrics(f32(res["halves"][0]), orc.gateup_split_fp32acc(f32(x), f32(wg), f32(wu)))
    assert m["rel_fro"] <= 1e-3 and m["scaled_max_abs"] <= 2.0 ** -7, m


def test_split_last_wave_is_used_at_the_7b_shape_and_matches(fsw, cuda_dev):
    """Down projection at the 7B prefill shape (256 pair tiles on 74 clusters = 3.46 waves) with the split along
    K forced (by default this shape takes the width split, which is bit-identical to the unsplit kernel);
    rows are compared with the CPU oracle and the whole output with the unsplit kernel."""
    M, d, F = 4096, 4096, 11008
    g = torch.Generator().manual_seed(5)
    h = torch.randn((M, F), generator=g).to(torch.bfloat16)
    wd = (torch.randn((d, F), generator=g) / F ** 0.5).to(torch.bfloat16)
    hd, wdd = h.to(cuda_dev), wd.to(cuda_dev)
    scratch = fsw.ops.gemm_scratch(cuda_dev)
    with env(FSWIGLU_TAIL_SPLITK="0"):
        o0 = fsw.ops.swiglu_down_bf16(hd, wdd, scratch=scratch)
    with env(FSWIGLU_TAIL_SPLITK="force"):
        o1 = fsw.ops.swiglu_down_bf16(hd, wdd, scratch=scratch)
        o2 = fsw.ops.swiglu_down_bf16(hd, wdd, scratch=scratch)
    healthy(fsw)
    assert torch.equal(o1, o2)
    assert not torch.equal(o0, o1), "the split was expected to change the summation order of the last wave"
    m = orc.error_metrics(f32(o1), f32(o0))
    assert m["rel_fro"] <= 1e-3 and m["scaled_max_abs"] <= 2.0 ** -7, m
    rows = [0, 127, 128, 255, 256, 2047, 3839, 3840, 3967, 4095]  # includes the last wave's tiles
    ref = orc.bf16_round(f32(h[rows]) @ f32(wd).T)
    m = orc.error_metrics(f32(o1[rows]), ref)
    assert m["rel_fro"] <= 1e-3 and m["scaled_max_abs"] <= 2.0 ** -7, m


# ------------------------------------------------------------------ full benchmark sizes
def _rows_to_check(M, n=64, seed=0):
    rng = np.random.default_rng(seed)
    edge = [r for r in (0, 1, 127, 128, 129, 255, 256, M - 257, M - 256, M - 129, M - 128, M - 31, M - 30, M - 2, M - 1)
            if 0 <= r < M]
    return sorted(set(edge + rng.choice(M, size=min(n, M), replace=False).tolist()))


def test_legacy_op_at_the_reference_benchmark_shape(fsw, cuda_dev):
    """bench_swiglu.py:84-91,106 of the reference: K = 8192, N = 2 * 28672 packed rows, M = 4096 tokens,
    C [M, N] with ldC = N.  Rows are checked against the CPU oracle with the kernel's rounding points."""
    M, K, N = 4096, 8192, 2 * 28672
    g = torch.Generator(device=cuda_dev).manual_seed(0)
    A = torch.randn((M, K), generator=g, device=cuda_dev, dtype=torch.float32).to(torch.bfloat16)
    B = (torch.randn((N, K), generator=g, device=cuda_dev, dtype=torch.float32) / K ** 0.5).to(torch.bfloat16)
    C = torch.zeros((M, N), dtype=torch.bfloat16, device=cuda_dev)
    fsw.ops.swiglu_fwd_bf16(M, N, K, A, K, B, K, C, N)
    healthy(fsw)
    out = C.flatten()[: M * N // 2].view(M, N // 2)
    assert bool((C.flatten()[M * N // 2:] == 0).all())
    rows = _rows_to_check(M, n=24)
    ref = orc.gateup_interleaved_fp32acc(f32(A[rows]), f32(B))
    m = orc.error_metrics(f32(out[rows]), ref)
    assert m["rel_fro"] <= 1e-3 and m["scaled_max_abs"] <= 2.0 ** -7, m


def test_70b_shape_full_size_single_gpu(fsw, cuda_dev):
    """Configuration 4 at full size on one GPU (M = 8192, d = 8192, F = 28672; K = 28672 = 448 k-blocks
    through the down kernel): tile-edge and random rows against the fp32 expression."""
    x, wg, wu, wd = fsw.inputs.make_config_inputs("c4_llama3_70b_prefill")
    out = fsw.ops.fused_swiglu_mlp_bf16(x.to(cuda_dev), wg.to(cuda_dev), wu.to(cuda_dev), wd.to(cuda_dev))
    healthy(fsw)
    rows = _rows_to_check(x.size(0), n=32)
    ref = orc.mlp_fp32(f32(x[rows]), f32(wg), f32(wu), f32(wd))
    m = orc.error_metrics(f32(out[rows]), ref)
    assert m["rel_fro"] <= 5e-3 and m["scaled_max_abs"] <= 8e-3, m


def test_ragged_13b_shard_full_size_single_gpu(fsw, cuda_dev):
    """One rank's shard of configuration 5 at full size: M = 32414 (mod 128 = 30), d = 5120, F/8 = 1728 (13.5
    column tiles), 1 % x50 outliers.  127 x 14 and 127 x 20 pair tiles: the two-SM kernel with ragged M and
    ragged N, and the split last wave.  All eight shards' fp32 partials are summed and rounded once."""
    x, wg, wu, wd = fsw.inputs.make_config_inputs("c5_ragged_13b")
    assert x.size(0) == 32414
    xd = x.to(cuda_dev)
    acc = torch.zeros((x.size(0), wd.size(0)), dtype=torch.float32, device=cuda_dev)
    for r in range(8):
        gs, us, ds = (t.to(cuda_dev) for t in fsw.pack.shard_mlp_weights(wg, wu, wd, 8, r))
        acc += fsw.ops.fused_swiglu_mlp_bf16(xd, gs, us, ds, out_dtype=torch.float32)
    healthy(fsw)
    rows = _rows_to_check(x.size(0), n=32)
    ref = orc.mlp_fp32(f32(x[rows]), f32(wg), f32(wu), f32(wd))
    m = orc.error_metrics(f32(acc[rows].to(torch.bfloat16)), ref)
    assert m["rel_fro"] <= 5e-3 and m["scaled_max_abs"] <= 8e-3, m
