"""Builds libwick_cuda.so in-tree with nvcc for sm_100a.

`--fmad=false` is part of the numerics contract, not a tuning knob: the CPU path the
kernels must match bit for bit never contracts a*b+c, and the kernels call fmaf
explicitly where the reference uses a fused NEON instruction.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from typing import List

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
LIB_PATH = os.path.join(_HERE, "libwick_cuda.so")
SOURCES = ["kernels_basic.cu", "kernels_gemv.cu", "kernels_attn.cu", "kernels_q6k.cu", "kernels_batch.cu", "kernels_sample.cu", "tp_comm.cu", "decode_mega.cu", "gemm_tc.cu", "argmax_noalloc.cu", "wick_cuda.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo", "--fmad=false",
    "-Xcompiler", "-fPIC,-Wall",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    for f in os.listdir(CSRC):
        if os.path.getmtime(os.path.join(CSRC, f)) > t:
            return True
    inc = os.path.join(_HERE, "..", "include", "wick_cuda.h")
    return os.path.getmtime(inc) > t or os.path.getmtime(__file__) > t


def build(force: bool = False, verbose: bool = False, extra: List[str] | None = None) -> str:
    if not force and not _stale():
        return LIB_PATH
    objdir = os.path.join(_HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    nvcc = _nvcc()
    env = dict(os.environ)
    # the environment may export CC/CXX pointing at a non-system compiler; nvcc wants the system g++
    ccbin = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    objs = []
    procs = []
    for src in SOURCES:
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        cmd = [nvcc, "-ccbin", ccbin, *NVCC_FLAGS, *(extra or []), "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((cmd, subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for cmd, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode:
            sys.stderr.write(out)
        if p.returncode:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
    link = [nvcc, "-ccbin", ccbin, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB_PATH, *objs]
    subprocess.check_call(link, env=env)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
