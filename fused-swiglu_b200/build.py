"""In-tree build of the native parts (sm_100a only).

  lib/libfswiglu.so                     the CUDA kernels + C ABI (nvcc, no torch)
  fused_mlp_module.<abi>.so             the torch extension with the reference's module and op
                                        names (g++, links libfswiglu.so through an $ORIGIN rpath)

Usage:  python fused-swiglu_b200/build.py [--lib-only] [--force] [-v]
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIB_DIR, "libfswiglu.so")
EXT = os.path.join(HERE, "fused_mlp_module" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-shared", "-Xcompiler", "-fPIC",
]


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError(f"build step failed: {' '.join(cmd[:3])} ...")
    if verbose and (res.stdout or res.stderr):
        print(res.stdout + res.stderr)


def lib_sources() -> list[str]:
    files = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith((".cu", ".cuh", ".h"))]
    files.append(os.path.join(os.path.dirname(HERE), "include", "fswiglu.h"))
    return files


def build_lib(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> str:
    srcs = lib_sources()
    if not force and _newer(LIB, srcs):
        return LIB
    os.makedirs(LIB_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, *NVCC_FLAGS]
    if ptxas_info:
        cmd += ["-Xptxas", "-v"]
    tmp = LIB + ".partial"
    cmd += ["-o", tmp] + [s for s in srcs if s.endswith(".cu")]
    _run(cmd, verbose or ptxas_info)
    os.replace(tmp, LIB)  # the library file is always a complete build
    return LIB


def build_ext(force: bool = False, verbose: bool = False) -> str:
    src = os.path.join(CSRC, "torch_bindings.cpp")
    if not force and _newer(EXT, [src, LIB]):
        return EXT
    from torch.utils import cpp_extension  # plumbing only: include paths and libraries

    inc = [f"-I{p}" for p in cpp_extension.include_paths()]
    inc += [f"-I{sysconfig.get_paths()['include']}", f"-I{os.path.join(os.path.dirname(HERE), 'include')}"]
    inc += ["-I/usr/local/cuda/include"]
    libdirs = cpp_extension.library_paths()
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-DTORCH_EXTENSION_NAME=fused_mlp_module",
           "-DTORCH_API_INCLUDE_EXTENSION_H", *inc, src, "-o", EXT + ".partial"]
    for d in libdirs:
        cmd += [f"-L{d}", f"-Wl,-rpath,{d}"]
    cmd += [f"-L{LIB_DIR}", "-Wl,-rpath,$ORIGIN/lib", "-lfswiglu", "-lc10", "-lc10_cuda", "-ltorch_cpu",
            "-ltorch_cuda", "-ltorch", "-ltorch_python"]
    _run(cmd, verbose)
    os.replace(EXT + ".partial", EXT)
    return EXT


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--lib-only", action="store_true")
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--ptxas-info", action="store_true")
    ap.add_argument("-v", "--verbose", action="store_true")
    a = ap.parse_args()
    print(build_lib(a.force, a.verbose, a.ptxas_info))
    if not a.lib_only:
        print(build_ext(a.force, a.verbose))


if __name__ == "__main__":
    main()
