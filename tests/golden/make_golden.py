"""Generate the golden fixtures in this directory.

The reference ships no known-answer vectors, so the fixtures are outputs of the reference's
own eager PyTorch expressions executed by PyTorch on CPU, on seeded inputs.  For the packed
gate-up op the expression is not restated here: lines 41-43 of the reference's numeric_tests.py
are READ FROM THAT FILE and executed as they stand (REFERENCE_DIR, default: the checkout the
build container mounts), so the stored outputs are the reference's own oracle, not a transcription
of it.  The whole-MLP expression (F.silu(x@Wg.T) * (x@Wu.T)) @ Wd.T is the one the benchmark's first
configuration prescribes (the reference itself stops after the gate).
Re-run with:   python tests/golden/make_golden.py        (needs the reference checkout)
bf16 tensors are stored as uint16 bit patterns, everything else as fp32.

  gateup_interleaved_small.npz   A [96,128], B [320,128] ~ U(+-1/sqrt(K)) (numeric_tests.py:8-10);
                                 out_eager_bf16 = the script's three lines on bf16 CPU tensors,
                                 out_fp32 = the same lines on fp32 copies of the inputs
  gateup_interleaved_unit.npz    same op, inputs ~ N(0,1) / N(0, 1/K), ragged sizes
  mlp_small.npz                  x [64,128], W_gate/W_up [192,128], W_down [128,192], out fp32
  mlp_ragged_outliers.npz        x [37,136] with 1 % entries x50, F = 200, out fp32
  mlp_c1_digest.json             digest (sums + sampled entries) of the fp32 output at the full
                                 configuration-1 size M=512, d=1024, F=2816, seed 0
"""
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "fused-swiglu_b200"))

from oracle import eager_reference as ref  # noqa: E402  (whole-MLP expression only)

REFERENCE_DIR = os.environ.get("FSWIGLU_REFERENCE_DIR", "/root/reference")
ORACLE_LINES = (41, 43)  # numeric_tests.py: C_torch = A @ B.T ; silu = F.silu(...) ; gated_torch = ...


def reference_oracle_source(reference_dir: str = REFERENCE_DIR) -> str:
    """Lines 41-43 of the reference's numeric_tests.py, dedented, exactly as they stand in the file."""
    import textwrap

    with open(os.path.join(reference_dir, "numeric_tests.py")) as f:
        lines = f.read().splitlines()
    return textwrap.dedent("\n".join(lines[ORACLE_LINES[0] - 1:ORACLE_LINES[1]])) + "\n"


def reference_gateup(A: torch.Tensor, B: torch.Tensor, source: str) -> torch.Tensor:
    """Execute the reference's own oracle lines on (A, B) and return what they call gated_torch."""
    import torch.nn.functional as F

    scope = {"A": A, "B": B, "F": F, "torch": torch}
    exec(compile(source, "numeric_tests.py:41-43", "exec"), scope)  # noqa: S102  (the reference's three lines)
    return scope["gated_torch"]

# inputs.py imports nothing native, load it without triggering the package's library load
import importlib.util  # noqa: E402

_spec = importlib.util.spec_from_file_location(
    "fsw_inputs", os.path.join(ROOT, "fused-swiglu_b200", "fused_swiglu_b200", "inputs.py"))
inputs = importlib.util.module_from_spec(_spec)
sys.modules["fsw_inputs"] = inputs
_spec.loader.exec_module(inputs)


def bits(t: torch.Tensor) -> np.ndarray:
    assert t.dtype == torch.bfloat16
    return t.view(torch.int16).numpy().view(np.uint16).copy()


def main() -> None:
    torch.set_num_threads(1)  # fixed summation order inside the CPU GEMMs
    src = reference_oracle_source()
    with open(os.path.join(HERE, "reference_oracle_lines.json"), "w") as f:
        json.dump({"file": "numeric_tests.py", "lines": list(ORACLE_LINES), "source": src}, f, indent=1)

    g = torch.Generator().manual_seed(1234)
    A = inputs.kaiming_uniform_bf16(96, 128, g)
    B = inputs.kaiming_uniform_bf16(320, 128, g)
    np.savez_compressed(os.path.join(HERE, "gateup_interleaved_small.npz"), A=bits(A), B=bits(B),
                        out_eager_bf16=bits(reference_gateup(A, B, src)),
                        out_fp32=reference_gateup(A.float(), B.float(), src).numpy())

    g = torch.Generator().manual_seed(4321)
    A = torch.randn((70, 200), generator=g).to(torch.bfloat16)
    B = (torch.randn((2 * 88, 200), generator=g) / 200 ** 0.5).to(torch.bfloat16)
    np.savez_compressed(os.path.join(HERE, "gateup_interleaved_unit.npz"), A=bits(A), B=bits(B),
                        out_eager_bf16=bits(reference_gateup(A, B, src)),
                        out_fp32=reference_gateup(A.float(), B.float(), src).numpy())

    x, wg, wu, wd = inputs.make_mlp_inputs(64, 128, 192, seed=0)
    np.savez_compressed(os.path.join(HERE, "mlp_small.npz"), x=bits(x), w_gate=bits(wg), w_up=bits(wu),
                        w_down=bits(wd), out_fp32=ref.mlp_eager_fp32(x, wg, wu, wd).numpy())

    x, wg, wu, wd = inputs.make_mlp_inputs(37, 136, 200, seed=5, outliers=True)
    np.savez_compressed(os.path.join(HERE, "mlp_ragged_outliers.npz"), x=bits(x), w_gate=bits(wg), w_up=bits(wu),
                        w_down=bits(wd), out_fp32=ref.mlp_eager_fp32(x, wg, wu, wd).numpy())

    x, wg, wu, wd = inputs.make_config_inputs("c1_cpu_small", seed=0)
    out = ref.mlp_eager_fp32(x, wg, wu, wd).double()
    digest = {
        "config": "c1_cpu_small", "seed": 0, "shape": list(out.shape),
        "x_bits_sum": int(bits(x).astype(np.int64).sum()),
        "w_gate_bits_sum": int(bits(wg).astype(np.int64).sum()),
        "w_down_bits_sum": int(bits(wd).astype(np.int64).sum()),
        "out_sum": float(out.sum()), "out_abs_sum": float(out.abs().sum()),
        "out_sq_sum": float((out * out).sum()), "out_abs_max": float(out.abs().max()),
        "sample_rows": list(range(0, 512, 64)), "sample_cols": list(range(0, 1024, 128)),
        "samples": out[0:512:64, 0:1024:128].tolist(),
    }
    with open(os.path.join(HERE, "mlp_c1_digest.json"), "w") as f:
        json.dump(digest, f, indent=1)
    print("fixtures written to", HERE)


if __name__ == "__main__":
    main()
