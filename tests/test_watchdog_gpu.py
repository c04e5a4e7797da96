"""The time-out path of the kernels, exercised without faulting, trapping or hanging anything: the wait
limit is lowered to a few milliseconds and one launch is made whose wait cannot be satisfied (an operand
copy that is never issued, a hand-over count that nothing reaches).  The wait runs out, the kernel unwinds
(copies and MMAs in flight drained, tensor memory freed, both CTAs of a pair leave together) and returns;
the host reads FSWIGLU_ERR_WATCHDOG with the site of the wait, the word clears, and the next ordinary call
gives bit-exact results, i.e. the context and the SMs' tensor memory are intact.
"""
import contextlib
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

SITE_MMA_FULL, SITE_PRODUCER_EMPTY, SITE_EPILOGUE_FULL, SITE_DECODE = 2, 1, 4, 7


@contextlib.contextmanager
def short_limit(capi, us):
    prev = capi.lib.fswiglu_set_wait_limit_us(us)
    try:
        yield
    finally:
        capi.lib.fswiglu_test_expire_next_wait(0)
        capi.lib.fswiglu_set_wait_limit_us(prev)


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


@pytest.mark.parametrize("kernel", ["one_sm", "two_sm", "two_sm_512", "small_batch"])
def test_a_wait_that_runs_out_is_reported_and_leaves_the_device_usable(cuda_dev, kernel):
    import fused_swiglu_b200 as fsw

    capi = fsw.capi
    M = 4 if kernel == "small_batch" else 300
    x, wg, wu, wd = (t.to(cuda_dev) for t in fsw.inputs.make_mlp_inputs(M, 520, 1096, seed=0))
    pair = {"two_sm": "force", "two_sm_512": ""}.get(kernel, "0")
    with env(FSWIGLU_PAIR=pair, FSWIGLU_QUAD="force" if kernel == "two_sm_512" else "0"):
        want = fsw.ops.fused_swiglu_mlp_bf16(x, wg, wu, wd)
        torch.cuda.synchronize()
        assert capi.device_status() == 0
        assert capi.lib.fswiglu_set_wait_limit_us(0) == 2_000_000  # the default limit
        with short_limit(capi, 3000):
            capi.lib.fswiglu_test_expire_next_wait(1)
            fsw.ops.fused_swiglu_mlp_bf16(x, wg, wu, wd)  # result undefined: one wait cannot be satisfied
            torch.cuda.synchronize()  # returns: the kernel unwound by itself
            word = capi.device_status()
        assert word != 0, "the time-out was not recorded"
        site, cta = word & 0xFF, (word >> 8) - 1
        if kernel == "small_batch":
            assert site == SITE_DECODE
        else:
            assert site in (SITE_MMA_FULL, SITE_PRODUCER_EMPTY, SITE_EPILOGUE_FULL) and cta in (0, 1)
        assert capi.device_status() == 0, "the status word must clear once it has been read"
        assert capi.lib.fswiglu_set_wait_limit_us(0) == 2_000_000
        # the next ordinary calls are bit-exact: context alive, tensor memory released, barriers fine
        for _ in range(2):
            got = fsw.ops.fused_swiglu_mlp_bf16(x, wg, wu, wd)
            torch.cuda.synchronize()
            assert torch.equal(got, want)
        assert capi.device_status() == 0
