"""The numpy oracle against the golden fixtures (outputs of the reference's eager PyTorch
expressions, see tests/golden/make_golden.py).  CPU only."""
import json
import os

import numpy as np
import pytest
import torch

from oracle import eager_reference as ref
from oracle import swiglu_oracle as orc


def load(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name))
    return {k: (orc.bf16_bits_to_f32(z[k]) if z[k].dtype == np.uint16 else z[k]) for k in z.files}


def test_bf16_round_matches_torch():
    g = torch.Generator().manual_seed(7)
    v = torch.cat([torch.randn(4096, generator=g) * 10.0 ** e for e in (-30, -3, 0, 3, 30)])
    v = torch.cat([v, torch.tensor([0.0, -0.0, float("inf"), -float("inf"), 1.00390625, 1.01171875, 3.3895e38])])
    want = v.to(torch.bfloat16).float().numpy()
    got = orc.bf16_round(v.numpy())
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert np.isnan(orc.bf16_round(np.array([np.nan], np.float32))).all()


def test_bf16_bits_roundtrip():
    bits = np.arange(0, 0x7F80, 37, dtype=np.uint16)  # finite positive bf16 values
    assert np.array_equal(orc.f32_to_bf16_bits(orc.bf16_bits_to_f32(bits)), bits)


@pytest.mark.parametrize("name", ["gateup_interleaved_small.npz", "gateup_interleaved_unit.npz"])
def test_packed_gateup_eager_bf16_matches_reference_lines(golden_dir, name):
    z = load(golden_dir, name)
    got = orc.gateup_interleaved_eager_bf16(z["A"], z["B"])
    want = z["out_eager_bf16"]
    # Every intermediate is rounded to bf16; numpy and torch may sum the K products in a different
    # order, which can move C across a bf16 rounding boundary, and that one-ulp change is rounded
    # again in the product: allow two bf16 ulps on a handful of entries, exact equality on the rest.
    diff = np.abs(got - want)
    two_ulp = np.abs(want) * 2.0 ** -6 + 1e-30
    assert (diff <= two_ulp).all()
    assert (diff > 0).mean() < 0.01


@pytest.mark.parametrize("name", ["gateup_interleaved_small.npz", "gateup_interleaved_unit.npz"])
def test_packed_gateup_fp32_matches_reference_lines(golden_dir, name):
    z = load(golden_dir, name)
    got = orc.gateup_interleaved_fp32acc(z["A"], z["B"], round_out=False)
    m = orc.error_metrics(got, z["out_fp32"])
    assert m["rel_fro"] < 1e-6, m


def test_packed_and_split_forms_agree(golden_dir):
    z = load(golden_dir, "gateup_interleaved_unit.npz")
    up, gate = z["B"][0::2], z["B"][1::2]
    a = orc.gateup_interleaved_fp32acc(z["A"], z["B"])
    b = orc.gateup_split_fp32acc(z["A"], gate, up)
    assert np.array_equal(a, b)


@pytest.mark.parametrize("name", ["mlp_small.npz", "mlp_ragged_outliers.npz"])
def test_mlp_fp32_matches_reference_expression(golden_dir, name):
    z = load(golden_dir, name)
    got = orc.mlp_fp32(z["x"], z["w_gate"], z["w_up"], z["w_down"])
    m = orc.error_metrics(got, z["out_fp32"])
    assert m["rel_fro"] < 1e-6, m


@pytest.mark.parametrize("name", ["mlp_small.npz", "mlp_ragged_outliers.npz"])
def test_bf16_pipeline_within_graded_tolerance(golden_dir, name):
    """The rounding points of the GPU path stay inside rel-Fro 5e-3 of the fp32 expression."""
    z = load(golden_dir, name)
    got = orc.mlp_bf16_pipeline(z["x"], z["w_gate"], z["w_up"], z["w_down"])
    m = orc.error_metrics(got, z["out_fp32"])
    assert m["rel_fro"] < 5e-3, m


def test_c1_digest(golden_dir):
    """Full configuration-1 size: seeded generator + oracle reproduce the committed digest."""
    from fused_swiglu_b200 import inputs

    with open(os.path.join(golden_dir, "mlp_c1_digest.json")) as f:
        dg = json.load(f)
    x, wg, wu, wd = inputs.make_config_inputs("c1_cpu_small", seed=0)
    bits = lambda t: t.view(torch.int16).numpy().view(np.uint16).astype(np.int64).sum()  # noqa: E731
    assert int(bits(x)) == dg["x_bits_sum"]
    assert int(bits(wg)) == dg["w_gate_bits_sum"]
    assert int(bits(wd)) == dg["w_down_bits_sum"]
    f32 = lambda t: t.float().numpy()  # noqa: E731
    out = orc.mlp_fp32(f32(x), f32(wg), f32(wu), f32(wd)).astype(np.float64)
    assert list(out.shape) == dg["shape"]
    assert abs(out.sum() - dg["out_sum"]) < 1e-3 * dg["out_abs_sum"] * 1e-3
    assert abs(np.abs(out).sum() - dg["out_abs_sum"]) < 1e-5 * dg["out_abs_sum"]
    assert abs((out * out).sum() - dg["out_sq_sum"]) < 1e-5 * dg["out_sq_sum"]
    samples = out[np.ix_(dg["sample_rows"], dg["sample_cols"])]
    assert np.allclose(samples, np.array(dg["samples"]), rtol=1e-4, atol=1e-6)


def test_eager_reference_matches_oracle_on_fresh_inputs():
    from fused_swiglu_b200 import inputs

    x, wg, wu, wd = inputs.make_mlp_inputs(33, 72, 104, seed=11)
    f32 = lambda t: t.float().numpy()  # noqa: E731
    got = orc.mlp_fp32(f32(x), f32(wg), f32(wu), f32(wd))
    want = ref.mlp_eager_fp32(x, wg, wu, wd).numpy()
    assert orc.error_metrics(got, want)["rel_fro"] < 1e-6


def test_tp_partials_sum_to_full():
    from fused_swiglu_b200 import inputs, pack

    x, wg, wu, wd = inputs.make_mlp_inputs(16, 64, 200, seed=3)
    f32 = lambda t: t.float().numpy()  # noqa: E731
    full = orc.mlp_bf16_pipeline(f32(x), f32(wg), f32(wu), f32(wd), round_out=False)
    for world in (1, 2, 3, 8):
        parts = orc.mlp_tp_partials(f32(x), f32(wg), f32(wu), f32(wd), world, pack.shard_bounds)
        assert orc.error_metrics(sum(parts), full)["rel_fro"] < 1e-6


def test_error_metrics_values():
    ref_a = np.array([[3.0, 4.0]])
    got = np.array([[3.0, 4.5]])
    m = orc.error_metrics(got, ref_a)
    assert m["max_abs"] == 0.5 and abs(m["rel_fro"] - 0.1) < 1e-12 and abs(m["scaled_max_abs"] - 0.125) < 1e-12


# ------------------------------------------------------------------ pinning to the reference's own file
def _bits(t):
    return t.view(torch.int16).numpy().view(np.uint16)


def _run_reference_lines(source, A, B):
    import torch.nn.functional as F

    scope = {"A": A, "B": B, "F": F, "torch": torch}
    exec(compile(source, "numeric_tests.py:41-43", "exec"), scope)  # noqa: S102
    return scope["gated_torch"]


@pytest.mark.parametrize("name", ["gateup_interleaved_small.npz", "gateup_interleaved_unit.npz"])
def test_fixtures_are_outputs_of_the_stored_reference_lines(golden_dir, name):
    """The committed outputs are what the reference's own three oracle lines (stored verbatim with their
    file and line numbers) produce on the committed inputs: bit for bit on bf16 tensors."""
    with open(os.path.join(golden_dir, "reference_oracle_lines.json")) as f:
        stored = json.load(f)
    assert stored["file"] == "numeric_tests.py" and stored["lines"] == [41, 43]
    z = np.load(os.path.join(golden_dir, name))
    A = torch.from_numpy(z["A"].view(np.int16).copy()).view(torch.bfloat16)
    B = torch.from_numpy(z["B"].view(np.int16).copy()).view(torch.bfloat16)
    torch.set_num_threads(1)
    got = _run_reference_lines(stored["source"], A, B)
    assert np.array_equal(_bits(got), z["out_eager_bf16"])
    got32 = _run_reference_lines(stored["source"], A.float(), B.float())
    assert np.allclose(got32.numpy(), z["out_fp32"], rtol=1e-6, atol=1e-9)
    # the restatement kept beside the oracle is the same computation
    assert np.array_equal(_bits(ref.gateup_interleaved_eager(A, B)), z["out_eager_bf16"])


def test_stored_lines_are_the_reference_files_lines():
    """Where the reference checkout is present (the build container), the stored lines must be exactly
    lines 41-43 of its numeric_tests.py, and the restatement in oracle/eager_reference.py must consist of
    the same three statements."""
    import importlib.util
    import inspect

    ref_dir = os.environ.get("FSWIGLU_REFERENCE_DIR", "/root/reference")
    if not os.path.exists(os.path.join(ref_dir, "numeric_tests.py")):
        pytest.skip("reference checkout not present on this machine")
    here = os.path.dirname(os.path.abspath(__file__))
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(here, "golden", "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    with open(os.path.join(here, "golden", "reference_oracle_lines.json")) as f:
        stored = json.load(f)
    assert mg.reference_oracle_source(ref_dir) == stored["source"]
    norm = lambda text: [" ".join(ln.split()) for ln in text.strip().splitlines() if ln.strip()]  # noqa: E731
    body = norm(inspect.getsource(ref.gateup_interleaved_eager))[1:]
    assert body[:2] == norm(stored["source"])[:2]
    assert body[2] == "return C_torch[:, ::2] * silu" and norm(stored["source"])[2] == "gated_torch = C_torch[:, ::2] * silu"
