"""Compiles the CUDA library for sm_100a into this directory (libkvarn_b200.so).

The shared object is built in-tree with plain nvcc: it has a C ABI and no Python or torch dependency.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libkvarn_b200.so")
SOURCES = ["kvb_api.cu", "kvb_append.cu", "kvb_attn.cu", "kvb_attn_general.cu", "kvb_prefill.cu", "kvb_record.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC"]
# per-file flags: the codec must not contract a*b+c (bit-exact codes), the attention kernels may
EXTRA = {"kvb_append.cu": ["-fmad=false"], "kvb_record.cu": ["-fmad=false"]}


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(HERE, "..", "include", "kvarn_b200.h"))
    objs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(CSRC, src.replace(".cu", ".o"))
        if force or _stale(o, [s] + headers):
            cmd = ["nvcc"] + ARCH + COMMON + EXTRA.get(src, []) + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
            subprocess.run(cmd, check=True)
        objs.append(o)
    if force or _stale(LIB, objs):
        subprocess.run(["nvcc"] + ARCH + ["-shared", "-o", LIB] + objs + ["-lcudart"], check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
