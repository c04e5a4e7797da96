"""Host-side logic that needs no GPU: weight layouts, shard bounds, seeded inputs, and that
the C-ABI library loads and exports every symbol include/fswiglu.h declares."""
import ctypes
import os
import re

import pytest
import torch

from fused_swiglu_b200 import capi, inputs, pack
from fused_swiglu_b200.tp import TensorParallelSwiGLU

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "fswiglu.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fswiglu_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = declared_symbols()
    assert len(names) >= 10
    raw = ctypes.CDLL(capi.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), f"{n} declared in include/fswiglu.h but not exported"
    assert sorted(capi.SIGNATURES) == names, "ctypes signature table and header disagree"


def test_status_strings_and_version():
    assert capi.status_string(capi.OK) == "ok"
    for code in range(-8, 0):
        assert capi.status_string(code) != "unknown status"
    assert capi.status_string(-99) == "unknown status"
    assert re.fullmatch(r"\d+\.\d+\.\d+", capi.version())


def test_workspace_sizes_are_host_arithmetic():
    assert capi.lib.fswiglu_workspace_bytes(0, 4096, 11008) == 0
    assert capi.lib.fswiglu_workspace_bytes(4096, 4096, 11008) >= 4096 * 11008 * 2
    assert capi.lib.fswiglu_host_workspace_bytes(4096, 4096, 11008) >= 2 * 4096 * 4096 * 2


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU failure mode")
def test_compute_calls_fail_loudly_without_a_gpu():
    """No CPU fallback: on a machine without an sm_100 device the entry points return an error."""
    buf = (ctypes.c_uint16 * 64)()
    p = ctypes.cast(buf, ctypes.c_void_p)
    rc = capi.lib.fswiglu_gateup_bf16(p, 8, p, 8, p, p, 8, 1, 8, 8, 0, None)
    assert rc == capi.ERR_NO_DEVICE
    with pytest.raises(capi.FswigluError):
        capi.check(rc, "fswiglu_gateup_bf16")


def test_ops_reject_cpu_and_wrong_dtype_tensors():
    from fused_swiglu_b200 import ops

    a = torch.zeros((4, 8), dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        ops.fused_swiglu_bf16(a, torch.zeros((8, 8), dtype=torch.bfloat16))
    with pytest.raises(RuntimeError, match="bfloat16"):
        ops.fused_swiglu_bf16(a.float(), torch.zeros((8, 8)))


def test_interleave_roundtrip():
    g = torch.Generator().manual_seed(0)
    up = torch.randn((10, 16), generator=g).to(torch.bfloat16)
    gate = torch.randn((10, 16), generator=g).to(torch.bfloat16)
    w13 = pack.interleave_up_gate(up, gate)
    assert w13.shape == (20, 16)
    assert torch.equal(w13[0::2], up) and torch.equal(w13[1::2], gate)
    u2, g2 = pack.split_up_gate(w13)
    assert torch.equal(u2, up) and torch.equal(g2, gate)
    with pytest.raises(ValueError):
        pack.split_up_gate(w13[:19])


@pytest.mark.parametrize("F,world", [(28672, 8), (13824, 8), (11008, 4), (200, 3), (8, 8), (14336, 1)])
def test_shard_bounds_partition(F, world):
    spans = [pack.shard_bounds(F, world, r) for r in range(world)]
    assert spans[0][0] == 0 and spans[-1][1] == F
    for (lo, hi), (lo2, _) in zip(spans, spans[1:]):
        assert hi == lo2 and lo <= hi
    for lo, hi in spans[:-1]:
        assert (hi - lo) % 8 == 0
    assert pack.shard_bounds(13824, 8, 0) == (0, 1728)


def test_shard_weights_shapes():
    wg = torch.arange(24 * 16, dtype=torch.float32).reshape(24, 16)
    wd = torch.arange(16 * 24, dtype=torch.float32).reshape(16, 24)
    g, u, dn = pack.shard_mlp_weights(wg, wg + 1, wd, 3, 1)
    assert g.shape == (8, 16) and dn.shape == (16, 8) and dn.is_contiguous()
    assert torch.equal(g, wg[8:16]) and torch.equal(dn, wd[:, 8:16])


def test_seeded_inputs_are_deterministic_and_shaped():
    a = inputs.make_mlp_inputs(8, 16, 24, seed=0)
    b = inputs.make_mlp_inputs(8, 16, 24, seed=0)
    for s, t in zip(a, b):
        assert torch.equal(s, t) and s.dtype == torch.bfloat16
    assert a[0].shape == (8, 16) and a[1].shape == (24, 16) and a[3].shape == (16, 24)
    assert float(a[1].float().std()) == pytest.approx(0.02, rel=0.2)
    c = inputs.make_mlp_inputs(8, 16, 24, seed=1)
    assert not torch.equal(a[0], c[0])


def test_ragged_batch_length_is_the_configured_32414_rows():
    assert int(inputs.ragged_lengths(0).sum()) == 32414
    assert 32414 % 128 == 30


def test_outliers_present():
    g = torch.Generator().manual_seed(0)
    x = inputs.make_x(256, 256, g, outliers=True).float()
    frac = float((x.abs() > 6).float().mean())
    assert 0.003 < frac < 0.02


def test_tp_slab_bounds_cover_rows():
    w = torch.zeros((8, 16))
    for mode in ("allreduce", "rs_ag"):
        tp = TensorParallelSwiGLU(w, w, torch.zeros((16, 8)), n_slabs=4, mode=mode,
                                  local_partial=lambda *a: None, round_fn=lambda s, d: None)
        for M in (1, 7, 100, 4096, 32414):
            b = tp.slab_bounds(M)
            assert b[0][0] == 0 and b[-1][1] == M
            assert all(x[1] == y[0] for x, y in zip(b, b[1:]))
            assert len(b) <= 4


def test_host_slab_planner_properties():
    """The planner of the host-buffer step: same structural guarantees as the device-resident one, and it never
    prefers fewer slabs than that one (the exposed copies only add to the cost of tall first and last slabs)."""
    from fused_swiglu_b200.tp import _host_timeline_us, plan_host_slabs, plan_slabs

    for (M, d, Fl, world) in [(8192, 8192, 3584, 8), (8192, 8192, 14336, 2), (32414, 5120, 1728, 8), (32414, 5120, 6912, 2),
                              (4096, 4096, 5504, 2), (1000, 4096, 1376, 8), (1, 64, 8, 2)]:
        rows = plan_host_slabs(M, d, Fl, world, 148)
        assert sum(rows) == M and all(r > 0 for r in rows) and len(rows) <= 8
        assert all(r % (8 * world) == 0 for r in rows[:-1])
        dev_rows = plan_slabs(M, d, Fl, world, 148)
        assert len(rows) >= len(dev_rows)
        assert _host_timeline_us(rows, d, Fl, world, 148) <= _host_timeline_us(dev_rows, d, Fl, world, 148) + 1e-9


def test_slab_planner_properties():
    from fused_swiglu_b200.tp import plan_slabs

    for (M, d, Fl, world) in [(8192, 8192, 3584, 8), (8192, 8192, 14336, 2), (32414, 5120, 1728, 8), (4096, 4096, 5504, 2),
                              (1000, 4096, 1376, 8), (1, 64, 8, 2)]:
        rows = plan_slabs(M, d, Fl, world, 132)
        assert sum(rows) == M and all(r > 0 for r in rows) and len(rows) <= 8
        assert all(r % (8 * world) == 0 for r in rows[:-1])
    # the measured optimum at the 70B shape on 8 GPUs
    assert plan_slabs(8192, 8192, 3584, 8, 132) == [7168, 1024]
    assert plan_slabs(512, 4096, 1376, 8, 132) == [512]


def test_bench_reference_arm_prints_one_json_line():
    import json
    import subprocess
    import sys

    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "2",
                          "--warmup", "1"], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-500:]
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    j = json.loads(lines[0])
    assert j["impl"] == "reference" and j["unit"] == "TFLOP/s" and j["value"] > 0
    assert j["cpu_baseline"]["kind"] == "port" and j["e2e"]["h2d_bytes_per_step"] == 0
    assert j["config"]["workload"] == "c4_llama3_70b_prefill"


def test_torch_extension_surface_loads_without_a_gpu():
    """The drop-in module imports on a CPU-only box and registers the reference's names and schemas
    (csrc/torch_bindings.cpp:31-50 of the reference); calling an op there fails loudly."""
    import fused_mlp_module

    for name in ("fused_swiglu_bf16", "swiglu_fwd_bf16", "fused_swiglu_gateup_bf16", "swiglu_down_bf16",
                 "fused_swiglu_mlp_bf16", "rms_scale"):
        assert callable(getattr(fused_mlp_module, name))
        assert hasattr(torch.ops.ASMLLM, name)
    assert "Tensor X, Tensor W1W3" in str(torch.ops.ASMLLM.fused_swiglu_bf16.default._schema)
    assert "int m, int n, int k, Tensor A, int ldA, Tensor B, int ldB, Tensor C, int ldC" in \
        str(torch.ops.ASMLLM.swiglu_fwd_bf16.default._schema)
    with pytest.raises(RuntimeError):
        fused_mlp_module.fused_swiglu_bf16(torch.zeros((4, 8), dtype=torch.bfloat16),
                                           torch.zeros((8, 8), dtype=torch.bfloat16))


def test_meta_implementations_and_module_shapes():
    """Shape-only dispatch (what fake-tensor tracing uses) and the nn.Module wrapper, on the meta device."""
    import fused_mlp_module  # noqa: F401
    from fused_swiglu_b200.module import FusedSwiGLUMLP

    bf = dict(dtype=torch.bfloat16, device="meta")
    x, wg, wd = torch.empty((12, 64), **bf), torch.empty((40, 64), **bf), torch.empty((64, 40), **bf)
    ops = torch.ops.ASMLLM
    assert ops.fused_swiglu_mlp_bf16(x, wg, wg, wd).shape == (12, 64)
    assert ops.fused_swiglu_gateup_bf16(x, wg, wg).shape == (12, 40)
    assert ops.fused_swiglu_bf16(x, torch.empty((80, 64), **bf)).shape == (12, 40)
    assert ops.swiglu_down_bf16(torch.empty((12, 40), **bf), wd, True).dtype == torch.float32
    assert ops.swiglu_fwd_bf16_out(12, 80, 64, x, 64, torch.empty((80, 64), **bf), 64, torch.empty((12, 80), **bf),
                                   80) is None
    assert "Tensor(a!) C" in str(ops.swiglu_fwd_bf16_out.default._schema)
    # the op with the reference's own schema declares no mutation, so it is deliberately not traceable
    with pytest.raises(NotImplementedError):
        ops.swiglu_fwd_bf16(12, 80, 64, x, 64, torch.empty((80, 64), **bf), 64, torch.empty((12, 80), **bf), 80)
    assert ops.rms_scale(x, 1e-6).shape == (12,) and ops.rms_scale(x, 1e-6).dtype == torch.float32
    assert ops.fused_swiglu_mlp_bf16(x, wg, wg, wd, x, ops.rms_scale(x), True).dtype == torch.float32
    mlp = FusedSwiGLUMLP(64, 40, device="meta")
    assert mlp(torch.empty((2, 3, 64), **bf)).shape == (2, 3, 64)
    assert [n for n, _ in mlp.named_parameters()] == ["gate_proj", "up_proj", "down_proj"]
    with pytest.raises(ValueError):
        FusedSwiGLUMLP(60, 40)
    lin = torch.nn.Linear(64, 40, bias=False)
    m2 = FusedSwiGLUMLP.from_linears(lin, torch.nn.Linear(64, 40, bias=False), torch.nn.Linear(40, 64, bias=False))
    assert m2.gate_proj.dtype == torch.bfloat16 and torch.equal(m2.gate_proj.float(), lin.weight.to(torch.bfloat16).float())


def test_pair_kernel_schedule_arithmetic(tmp_path):
    """The work list of the two-SM GEMM kernel and the plan of its split last wave are plain integer
    code shared by host and device (csrc/pair_schedule.cuh): compile the checker with g++ and run it."""
    import subprocess

    exe = tmp_path / "check_pair_schedule"
    src = os.path.join(ROOT, "tests", "native", "check_pair_schedule.cpp")
    inc = os.path.join(ROOT, "fused-swiglu_b200", "csrc")
    subprocess.run(["g++", "-O1", "-std=c++17", f"-I{inc}", src, "-o", str(exe)], check=True)
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and res.stdout.startswith("ok "), res.stdout[-400:]


def test_host_pipeline_slab_plan(tmp_path):
    """The row slabs of the host-buffer pipeline (csrc/host_slabs.h) for every batch size up to 70 000 rows and
    a sweep beyond: contiguous, non-empty, covering, never more than the pipeline has events for."""
    import subprocess

    exe = tmp_path / "check_host_slabs"
    src = os.path.join(ROOT, "tests", "native", "check_host_slabs.cpp")
    inc = os.path.join(ROOT, "fused-swiglu_b200", "csrc")
    subprocess.run(["g++", "-O1", "-std=c++17", f"-I{inc}", src, "-o", str(exe)], check=True)
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and res.stdout.startswith("ok "), res.stdout[-400:]


def test_graph_capture_traces_through_the_ops():
    """torch.compile(fullgraph=True) must trace the module and the alias-annotated launcher without a graph
    break; on a CPU-only machine the captured graph then fails at run time, with the dispatcher's missing
    CPU kernel error and nothing else (the GPU suite runs the same graphs for real)."""
    import fused_mlp_module  # noqa: F401
    from fused_swiglu_b200.module import FusedNormSwiGLUBlock, FusedSwiGLUMLP

    if torch.cuda.is_available():
        pytest.skip("covered with real tensors by the GPU suite")
    bf = dict(dtype=torch.bfloat16)
    x = torch.zeros((2, 3, 64), **bf)
    for mod in (FusedSwiGLUMLP(64, 40), FusedNormSwiGLUBlock(64, 40)):
        torch._dynamo.reset()
        with pytest.raises(NotImplementedError, match="'CPU' backend"):
            torch.compile(mod, fullgraph=True, backend="aot_eager")(x)

    def launch(A, B, C):
        torch.ops.ASMLLM.swiglu_fwd_bf16_out(12, 80, 64, A, 64, B, 64, C, 80)
        return C * 2

    torch._dynamo.reset()
    with pytest.raises(NotImplementedError, match="'CPU' backend"):
        torch.compile(launch, fullgraph=True, backend="aot_eager")(torch.zeros((12, 64), **bf), torch.zeros((80, 64), **bf),
                                                                    torch.zeros((12, 80), **bf))
