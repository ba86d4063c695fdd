"""Builds libb200moe.so (hand-written sm_100a CUDA + the C ABI) in-tree with nvcc."""
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libb200moe.so")
SOURCES = ["api.cu", "router.cu", "permute.cu", "qmm_decode.cu", "qmm_prefill.cu", "misc.cu", "ep.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc():
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _deps_mtime():
    m = 0.0
    for root in (CSRC, os.path.join(HERE, "..", "include")):
        for f in os.listdir(root):
            m = max(m, os.path.getmtime(os.path.join(root, f)))
    return m


def build(force=False, verbose=False):
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _deps_mtime():
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    flags = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-ccbin", "/usr/bin/g++"] + ARCH
    if verbose:
        flags += ["-Xptxas", "-v"]
    if os.environ.get("B200_DEV"):      # development build: self-timing and debug switches compiled in
        flags += ["-DB200_DEV"]

    def one(src):
        obj = os.path.join(OBJ, src.replace(".cu", ".o"))
        r = subprocess.run([nvcc, *flags, "-c", os.path.join(CSRC, src), "-o", obj], capture_output=True, text=True)
        return src, obj, r

    objs = []
    with ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        for src, obj, r in ex.map(one, SOURCES):
            if verbose or r.returncode:
                sys.stderr.write(r.stdout + r.stderr)
            if r.returncode:
                raise RuntimeError(f"nvcc failed on {src}")
            objs.append(obj)
    subprocess.run([nvcc, "-shared", "-o", LIB, *objs, "-cudart", "static", "-ccbin", "/usr/bin/g++", *ARCH], check=True)
    return LIB


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv))
