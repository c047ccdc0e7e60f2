"""Builds libflagcx_noalloc.so: the allocation-free RMSNorm backward entry point
(csrc/rmsnorm_bwd_noalloc.cu), a plain C library without any torch dependency."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc", "rmsnorm_bwd_noalloc.cu")
HDR = os.path.join(HERE, "csrc", "rmsnorm_bwd_noalloc.h")
LIB = os.path.join(HERE, "libflagcx_noalloc.so")


def build(verbose: bool = False) -> str:
    if os.path.exists(LIB) and os.path.getmtime(LIB) >= max(os.path.getmtime(SRC), os.path.getmtime(HDR)):
        return LIB
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    cmd = [nvcc, "-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a", "-shared",
           "-Xcompiler", "-fPIC", "-cudart", "static", SRC, "-o", LIB]
    res = subprocess.run(cmd, capture_output=not verbose, text=True)
    if res.returncode != 0:
        sys.stderr.write((res.stdout or "") + (res.stderr or ""))
        raise RuntimeError("building libflagcx_noalloc.so failed")
    return LIB
