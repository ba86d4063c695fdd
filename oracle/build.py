"""Build recipe for the CPU oracle (test infrastructure; never imported by the shipped package).

The reference cannot be compiled in this environment (it is a Rust binding over an MLX
submodule that is absent), so there is no `oracle/_ref` build: the oracle is a restatement.
"""
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "moe_oracle.cpp")
LIB = os.path.join(HERE, "libmoe_oracle.so")


def _cxx():
    for cand in ("/usr/bin/g++", shutil.which("g++") or ""):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("no g++ found for the oracle build")


def build(force=False):
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    cmd = [_cxx(), "-O3", "-march=x86-64-v3", "-fopenmp", "-fPIC", "-std=c++17", "-ffp-contract=off",
           "-Wall", "-Wextra", "-shared", "-o", LIB, SRC]
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
