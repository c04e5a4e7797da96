"""Run one of the reference project's own scripts (numeric_tests.py, bench_swiglu.py) UNCHANGED
against this library.

    python fused-swiglu_b200/run_reference_script.py /path/to/Fused-SwiGLU/numeric_tests.py

What it sets up, and nothing else: this directory goes to the front of sys.path (so that
`import fused_mlp_module` finds the extension built here, which exports the reference's module
and function names, csrc/torch_bindings.cpp:31-36 there), the script's own directory comes next
(bench_swiglu.py:7 imports its sibling unsloth_no_bs.py), and compat/ is appended at the END of
sys.path, behind site-packages, so that its import-only stand-ins for xformers, fused_swiglu and
matplotlib never shadow a real installation.  The script then runs as __main__ in the current
working directory (bench_swiglu.py:121 writes its CSV there).
"""
from __future__ import annotations

import os
import runpy
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
COMPAT = os.path.join(os.path.dirname(HERE), "compat")


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    script = os.path.abspath(sys.argv[1])
    sys.path.insert(0, os.path.dirname(script))
    sys.path.insert(0, HERE)
    sys.path.append(COMPAT)
    sys.argv = [script] + sys.argv[2:]
    runpy.run_path(script, run_name="__main__")


if __name__ == "__main__":
    main()
