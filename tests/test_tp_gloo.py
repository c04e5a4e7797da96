"""Tensor-parallel host logic with CPU ranks over gloo (world_size 2 and 3): sharding, slab
schedule, collective and the single final rounding.  The rank-local GEMMs are stood in for by
the numpy oracle here (the CUDA kernels themselves are covered by the gpu-marked tests); what is
under test is everything around them.  A rank that dies makes the others fail with an error
instead of hanging."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _oracle_partial(x, wg, wu, wd, out_f32, ws):
    from oracle import swiglu_oracle as orc

    f = lambda t: t.float().numpy()  # noqa: E731
    out_f32.copy_(torch.from_numpy(orc.mlp_bf16_pipeline(f(x), f(wg), f(wu), f(wd), round_out=False)))


def _round(src, dst):
    dst.copy_(src.to(torch.bfloat16))


def _worker(rank, world, port, mode, M, fail_rank, q):
    for p in (ROOT, os.path.join(ROOT, "fused-swiglu_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import datetime

    from fused_swiglu_b200 import inputs
    from fused_swiglu_b200.tp import TensorParallelSwiGLU
    from oracle import swiglu_oracle as orc

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        x, wg, wu, wd = inputs.make_mlp_inputs(M, 64, 200, seed=2)
        tp = TensorParallelSwiGLU.from_full(wg, wu, wd, torch.device("cpu"), n_slabs=3, mode=mode,
                                            local_partial=_oracle_partial, round_fn=_round)
        if rank == fail_rank:
            os._exit(17)  # dies between steps, nothing in flight
        out = tp.forward(x)
        f = lambda t: t.float().numpy()  # noqa: E731
        ref = orc.mlp_fp32(f(x), f(wg), f(wu), f(wd))
        m = orc.error_metrics(f(out), ref)
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out)
        same = all(torch.equal(g, out) for g in gathered)
        # the rows each rank hands back in the host-buffer step cover the result exactly once, in this mode and
        # in the slab-wise ownership of the push mode (pure index arithmetic, no GPU needed)
        push = TensorParallelSwiGLU.from_full(wg, wu, wd, torch.device("cpu"), n_slabs=3, mode="push",
                                              local_partial=_oracle_partial, round_fn=_round)
        for inst, rows in ((tp, M), (push, M), (push, 8192), (push, 777)):
            mine = inst.owned_rows(rows)
            everyone = [None] * world
            dist.all_gather_object(everyone, mine)
            covered = sorted(r for ranges in everyone for g0, g1 in ranges for r in range(g0, g1))
            same = same and covered == list(range(rows))
        q.put((rank, "ok", m["rel_fro"], same, tuple(out.shape)))
    except Exception as e:  # noqa: BLE001
        q.put((rank, "error", repr(e)[:200], False, ()))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def _run(world, mode, M, fail_rank=-1):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, M, fail_rank, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = []
    expected = world - (1 if fail_rank >= 0 else 0)
    for _ in range(expected):
        results.append(q.get(timeout=120))
    for p in procs:
        p.join(timeout=60)
    return sorted(results), [p.exitcode for p in procs]


@pytest.mark.parametrize("world,mode,M", [(2, "allreduce", 50), (2, "rs_ag", 50), (3, "rs_ag", 37), (2, "allreduce", 1)])
def test_tp_forward_matches_oracle(world, mode, M):
    results, codes = _run(world, mode, M)
    assert codes == [0] * world
    for rank, status, rel_fro, same, shape in results:
        assert status == "ok", results
        assert shape == (M, 64)
        assert rel_fro < 5e-3
        assert same, "ranks disagree on the reduced output"


def test_tp_rank_failure_is_an_error_not_a_hang():
    results, codes = _run(2, "allreduce", 20, fail_rank=1)
    assert codes[1] == 17
    (rank, status, msg, _, _), = results
    assert rank == 0 and status == "error", results
