"""Build libm2b200.so for sm_100a with nvcc (cross-compiles without a GPU).

    python -m m2_b200.csrc.build [--verbose]
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(os.path.dirname(HERE), "libm2b200.so")
SOURCES = ["m2_b200.cu"]   # single translation unit that includes the other .cu parts
PARTS = ["abi.cu", "filter.cu", "longconv_simt.cu", "longconv_tc.cu", "longconv_tcl.cu", "longconv_tz.cu", "longconv.cu",
         "gemm_tc.cu", "linear_tc.cu", "glu_pair.cu", "gemm_simt.cu", "selftest.cu", "common.cuh", "tc_common.cuh", "m2_b200.cu",
         os.path.join("..", "..", "include", "m2_b200.h")]


def needs_build():
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    return any(os.path.getmtime(os.path.join(HERE, p)) > t for p in PARTS
               if os.path.exists(os.path.join(HERE, p)))


def build(verbose=False, force=False):
    if not force and not needs_build():
        return OUT
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-shared", "-Xcompiler", "-fPIC", "-o", OUT] + SOURCES
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    res = subprocess.run(cmd, cwd=HERE, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libm2b200.so")
    return OUT


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv, force=True))
