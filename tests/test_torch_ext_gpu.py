"""The drop-in boundary: `fused_mlp_module` (pybind) and `torch.ops.ASMLLM.*` (dispatcher) with the
reference's names and schemas (csrc/torch_bindings.cpp:31-50), exercised the way the reference's
own scripts do it, but with assertions (the scripts only print)."""
import math

import numpy as np
import pytest
import torch
import torch.nn.functional as F
from torch.nn import init

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mod(cuda_dev):
    import fused_mlp_module

    return fused_mlp_module


def test_module_and_dispatcher_surface(mod):
    for name in ("fused_swiglu_bf16", "swiglu_fwd_bf16", "fused_swiglu_gateup_bf16", "swiglu_down_bf16",
                 "fused_swiglu_mlp_bf16"):
        assert hasattr(mod, name)
        assert hasattr(torch.ops.ASMLLM, name)
    schema = str(torch.ops.ASMLLM.fused_swiglu_bf16.default._schema)
    assert "Tensor X, Tensor W1W3" in schema and "-> Tensor" in schema
    schema = str(torch.ops.ASMLLM.swiglu_fwd_bf16.default._schema)
    assert "int m, int n, int k, Tensor A, int ldA, Tensor B, int ldB, Tensor C, int ldC" in schema


@pytest.mark.parametrize("MNK", [256, 1024, 2048])
def test_numeric_tests_script_logic(mod, cuda_dev, MNK):
    """numeric_tests.py:27-52 with thresholds: kaiming-uniform bf16 operands, bf16-eager oracle on the
    GPU, the three statistics the script prints.  The oracle's own bf16 intermediates dominate the
    difference (about 3.7e-3 rel-Fro); absolute errors are ~1e-6 because |A|,|B| <= 1/sqrt(K)."""
    torch.manual_seed(0)
    M = N = K = MNK
    rels, maxs = [], []
    for _ in range(3):
        A = init.kaiming_uniform_(torch.randn((M, K), device=cuda_dev, dtype=torch.bfloat16), a=math.sqrt(5))
        B = init.kaiming_uniform_(torch.randn((N, K), device=cuda_dev, dtype=torch.bfloat16), a=math.sqrt(5))
        C_torch = A @ B.T
        silu = F.silu(C_torch[:, 1::2])
        gated_torch = C_torch[:, ::2] * silu
        gated_mine = mod.fused_swiglu_bf16(A, B)
        diff = gated_mine - gated_torch
        maxs.append(diff.abs().max().item())
        rels.append(diff.norm(p="fro").item() / gated_torch.norm(p="fro").item())
    assert np.mean(rels) <= 5e-3, rels
    assert max(maxs) <= 2e-2, maxs


def test_bench_script_call_pattern(mod, cuda_dev):
    """bench_swiglu.py:87-91,106: C is [M, N] zeros, ldC = N."""
    M, K, N = 512, 1024, 2 * 768
    A = torch.randn((M, K), dtype=torch.bfloat16, device=cuda_dev)
    B = torch.randn((N, K), dtype=torch.bfloat16, device=cuda_dev) / 32
    C = torch.zeros((M, N), dtype=torch.bfloat16, device=cuda_dev)
    assert mod.swiglu_fwd_bf16(M, N, K, A, K, B, K, C, N) is None
    want = mod.fused_swiglu_bf16(A, B)
    assert torch.equal(C.flatten()[: M * N // 2].view(M, N // 2), want)
    torch.ops.ASMLLM.swiglu_fwd_bf16(M, N, K, A, K, B, K, C, N)
    assert torch.equal(torch.ops.ASMLLM.fused_swiglu_bf16(A, B), want)


def test_full_mlp_op_matches_ctypes_path(mod, cuda_dev):
    import fused_swiglu_b200 as fsw

    x, wg, wu, wd = (t.to(cuda_dev) for t in fsw.inputs.make_mlp_inputs(300, 256, 520, seed=2))
    a = mod.fused_swiglu_mlp_bf16(x, wg, wu, wd)
    b = fsw.ops.fused_swiglu_mlp_bf16(x, wg, wu, wd)
    assert torch.equal(a, b)
    h = mod.fused_swiglu_gateup_bf16(x, wg, wu)
    assert torch.equal(mod.swiglu_down_bf16(h, wd), a)
    assert mod.swiglu_down_bf16(h, wd, True).dtype == torch.float32
    assert fsw.capi.device_status() == 0


def test_dtype_errors_are_runtime_errors(mod, cuda_dev):
    A = torch.zeros((8, 8), device=cuda_dev)
    with pytest.raises(RuntimeError, match="bfloat16"):
        mod.fused_swiglu_bf16(A, A)
    with pytest.raises(RuntimeError):
        mod.fused_swiglu_bf16(A.bfloat16().cpu(), A.bfloat16().cpu())


def test_module_wrapper_matches_the_op(mod, cuda_dev):
    import fused_swiglu_b200 as fsw
    from fused_swiglu_b200.module import FusedSwiGLUMLP

    x, wg, wu, wd = (t.to(cuda_dev) for t in fsw.inputs.make_mlp_inputs(6 * 50, 256, 520, seed=21))
    mlp = FusedSwiGLUMLP(256, 520, device=cuda_dev)
    with torch.no_grad():
        mlp.gate_proj.copy_(wg)
        mlp.up_proj.copy_(wu)
        mlp.down_proj.copy_(wd)
    got = mlp(x.view(6, 50, 256))
    want = mod.fused_swiglu_mlp_bf16(x, wg, wu, wd)
    assert got.shape == (6, 50, 256) and torch.equal(got.reshape(-1, 256), want)
    assert fsw.capi.device_status() == 0
