"""Builds the CPU oracle shared object (test infrastructure, never part of the product path).

`python oracle/build.py` compiles oracle/gemma4_oracle.cpp with g++ -O3 and OpenMP into
oracle/liboxg4_oracle.so. AVX2+FMA is the instruction-set floor so that an object built on one
x86-64 host still loads on another.

The reference is Rust compiled through cuda-oxide; none of its sources can be built with gcc, so
there is no oracle/_ref build of the reference itself.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "gemma4_oracle.cpp")
OUT = os.path.join(HERE, "liboxg4_oracle.so")


def build_oracle(force: bool = False) -> str:
    if (not force and os.path.exists(OUT)
            and os.path.getmtime(OUT) >= os.path.getmtime(SRC)):
        return OUT
    cmd = ["g++", "-O3", "-std=c++17", "-fPIC", "-shared", "-fopenmp", "-mavx2", "-mfma",
           "-fno-math-errno", "-o", OUT, SRC]
    subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
