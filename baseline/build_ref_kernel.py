"""Build the reference project's own CUDA kernel for sm_100a, as a same-box GPU baseline.

The reference ships an sm_80-only build script and an un-vendored CUTLASS submodule; its
single translation unit (csrc/SwiGLU/swiglu.cu) and its binding file (csrc/torch_bindings.cpp)
compile unchanged for sm_100a against the CUTLASS/CuTe headers that ship inside the
flashinfer wheel.  This script compiles those two files WHERE THEY LIE (nothing is copied)
into   baseline/_ref/fused_mlp_module_ref<abi>.so   (git-ignored).  The module is only ever
imported by bench.py's baseline subprocess and by nothing that ships; it registers the same
dispatcher namespace as this repository's own extension, so the two are never loaded into one
process.

Usage:  python baseline/build_ref_kernel.py [--reference /path/to/Fused-SwiGLU] [--force]
The kernel template takes about six minutes to compile.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
MODULE = "fused_mlp_module_ref"


def cutlass_include() -> str | None:
    for p in sys.path:
        cand = os.path.join(p, "flashinfer", "data", "cutlass", "include")
        if os.path.isdir(cand):
            return cand
    return None


def target() -> str:
    return os.path.join(OUT_DIR, MODULE + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))


def build(reference: str, force: bool = False, verbose: bool = True) -> str | None:
    out = target()
    if os.path.exists(out) and not force:
        return out
    cu = os.path.join(reference, "csrc", "SwiGLU", "swiglu.cu")
    cpp = os.path.join(reference, "csrc", "torch_bindings.cpp")
    cutlass = cutlass_include()
    if not (os.path.exists(cu) and os.path.exists(cpp) and cutlass):
        return None
    from torch.utils import cpp_extension

    os.makedirs(OUT_DIR, exist_ok=True)
    inc = [f"-I{p}" for p in cpp_extension.include_paths()]
    inc += [f"-I{sysconfig.get_paths()['include']}", f"-I{cutlass}",
            f"-I{os.path.join(os.path.dirname(cutlass), 'tools', 'util', 'include')}", "-I/usr/local/cuda/include"]
    defs = [f"-DTORCH_EXTENSION_NAME={MODULE}", "-DTORCH_API_INCLUDE_EXTENSION_H"]
    obj_cu = os.path.join(OUT_DIR, "swiglu.o")
    obj_cpp = os.path.join(OUT_DIR, "torch_bindings.o")
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    steps = [
        # the reference's own nvcc flags (setup.py:28-37) with the architecture replaced
        [nvcc, "-c", cu, "-o", obj_cu, "-O3", "--use_fast_math", "--expt-relaxed-constexpr", "-std=c++17",
         "-gencode", "arch=compute_100a,code=sm_100a", "--compiler-options", "-fPIC", "-lineinfo",
         "-Xptxas", "-dlcm=cg", "-w", *inc, *defs],
        ["g++", "-c", cpp, "-o", obj_cpp, "-O3", "-std=c++17", "-fPIC", "-w", *inc, *defs],
    ]
    link = ["g++", "-shared", obj_cu, obj_cpp, "-o", out]
    for d in cpp_extension.library_paths():
        link += [f"-L{d}", f"-Wl,-rpath,{d}"]
    link += ["-L/usr/local/cuda/lib64", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
             "-ltorch_python", "-lcudart"]
    for cmd in steps + [link]:
        if verbose:
            print(" ".join(cmd[:4]), "...", flush=True)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout[-4000:] + res.stderr[-4000:])
            return None
    for o in (obj_cu, obj_cpp):
        os.remove(o)
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("FSWIGLU_REFERENCE_DIR", "/root/reference"))
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    out = build(a.reference, a.force)
    print(out if out else "reference kernel not built (sources or CUTLASS headers missing, or a compile step failed)")
    sys.exit(0 if out else 1)


if __name__ == "__main__":
    main()
