"""Compiles the CUDA library (csrc/oxg4.cu -> liboxg4.so) for sm_100a, in-tree.

`python oxide-beta_b200/build.py [--force] [--verbose]`. nvcc cross-compiles without a GPU. The
shared object sits next to this file so that it travels with the source tree; it is never
installed into site-packages.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "liboxg4.so")
SOURCES = ["oxg4.cu"]


def _newest_source() -> float:
    # every file under csrc/ is compiled into the one translation unit: any edit triggers a rebuild
    files = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh", ".h"))]
    files.append(os.path.join(os.path.dirname(HERE), "include", "oxg4.h"))
    return max(os.path.getmtime(f) for f in files if os.path.exists(f))


def build_library(force: bool = False, verbose: bool = False) -> str:
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= _newest_source():
        return OUT
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-shared", "-Xcompiler", "-fPIC", "--threads", "4", "-cudart", "static"]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES] + ["-o", OUT]
    subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
