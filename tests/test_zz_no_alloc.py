"""fswiglu_mlp_bf16_static: the whole-MLP call for hosts that must not allocate device memory
(a server that gave the whole GPU to its own pool at start-up, a latency-critical loop that cannot
afford the device-wide synchronisation of cudaMalloc).  Its hidden activations live in a fixed
32 MiB array inside the library instead of a caller workspace.

Checked here, through the C ABI: the result is bit-identical to fswiglu_mlp_bf16 on two calls in a
row with different inputs and sizes (the array keeps the first call's contents, which must not leak
into the second), a warm call leaves the driver's free-memory figure and torch's allocator counters
unchanged, its time-out word can be read, and a problem larger than the array is refused with
FSWIGLU_ERR_TOO_LARGE.
The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _vp(t):
    return ctypes.c_void_p(t.data_ptr())


def _static_mlp(lib, x, wg, wu, wd, out_dtype_code, out):
    M, d = x.shape
    F = wg.size(0)
    return lib.fswiglu_mlp_bf16_static(_vp(x), d, _vp(wg), _vp(wu), d, _vp(wd), F, _vp(out), d, out_dtype_code,
                                       M, d, F, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_static_scratch_entry_point_matches_workspace_entry_point(cuda_dev):
    import fused_swiglu_b200 as fsw

    lib, capi = fsw.capi.lib, fsw.capi
    # two calls in a row: a larger problem first, then a smaller one with other data, then fp32 output
    cases = [(300, 520, 1096, 0, torch.bfloat16), (77, 520, 1096, 1, torch.bfloat16), (129, 256, 264, 2, torch.float32)]
    for M, d, F, seed, dtype in cases:
        x, wg, wu, wd = (t.to(cuda_dev) for t in fsw.inputs.make_mlp_inputs(M, d, F, seed=seed))
        want = fsw.ops.fused_swiglu_mlp_bf16(x, wg, wu, wd, out_dtype=dtype)
        got = torch.full((M, d), float("nan"), dtype=dtype, device=cuda_dev)
        code = capi.OUT_BF16 if dtype == torch.bfloat16 else capi.OUT_F32
        rc = _static_mlp(lib, x, wg, wu, wd, code, got)
        assert rc == capi.OK, capi.status_string(rc)
        torch.cuda.synchronize()
        # same kernels, same tile schedule, same rounding points: the tolerance is zero
        assert torch.equal(got, want), f"case M={M} d={d} F={F}"
    # the time-out word of this entry point sits next to its array; both status calls report it
    assert capi.static_status() == 0
    assert capi.device_status() == 0


def test_static_scratch_entry_point_allocates_nothing(cuda_dev):
    """What the entry point is for: a warm call must not take device memory from anybody.  Checked on
    both levels: the driver's free-memory figure (cudaMemGetInfo) and torch's caching-allocator counters
    are the same before and after a call, and so is the launch path's own bookkeeping."""
    import fused_swiglu_b200 as fsw

    lib, capi = fsw.capi.lib, fsw.capi
    x, wg, wu, wd = (t.to(cuda_dev) for t in fsw.inputs.make_mlp_inputs(300, 520, 1096, seed=0))
    out = torch.empty((300, 520), dtype=torch.bfloat16, device=cuda_dev)
    assert _static_mlp(lib, x, wg, wu, wd, capi.OUT_BF16, out) == capi.OK  # first call on the device: set-up
    assert capi.static_status() == 0
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(cuda_dev)
    stats_before = torch.cuda.memory_stats(cuda_dev)
    for _ in range(3):
        assert _static_mlp(lib, x, wg, wu, wd, capi.OUT_BF16, out) == capi.OK
    torch.cuda.synchronize()
    assert capi.static_status() == 0
    free_after, _ = torch.cuda.mem_get_info(cuda_dev)
    stats_after = torch.cuda.memory_stats(cuda_dev)
    assert free_after == free_before, "device memory was taken during a warm call"
    for key in ("allocation.all.allocated", "segment.all.allocated", "reserved_bytes.all.current"):
        assert stats_after[key] == stats_before[key], key


def test_static_scratch_entry_point_refuses_oversized_problems(cuda_dev):
    import fused_swiglu_b200 as fsw

    lib, capi = fsw.capi.lib, fsw.capi
    buf = torch.zeros(64, dtype=torch.bfloat16, device=cuda_dev)
    p = _vp(buf)
    # M * F * 2 bytes = 32 MiB + 2 * F: one row too many
    F = 16384
    M = (32 << 20) // 2 // F + 1
    rc = lib.fswiglu_mlp_bf16_static(p, 4096, p, p, 4096, p, F, p, 4096, 0, M, 4096, F, None)
    assert rc == capi.ERR_TOO_LARGE
    assert "32 MiB" in capi.status_string(rc)
    # the largest size that fits is accepted as far as the size check goes (bad pointers are caught next)
    rc = lib.fswiglu_mlp_bf16_static(None, 4096, p, p, 4096, p, F, p, 4096, 0, M - 1, 4096, F, None)
    assert rc == capi.ERR_BAD_ARG
    # empty batch stays a no-op
    assert lib.fswiglu_mlp_bf16_static(None, 8, None, None, 8, None, 8, None, 8, 0, 0, 8, 8, None) == capi.OK
