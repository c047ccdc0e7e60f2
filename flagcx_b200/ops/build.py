"""Compiles the fused-op CUDA extension in-tree for sm_100a."""
from __future__ import annotations

import glob
import os
import shutil

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
NAME = "_flagcx_ops_C"
SOURCES = ["fused_elementwise.cu"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a", "--use_fast_math"]


def built_path() -> str | None:
    hits = glob.glob(os.path.join(HERE, NAME + "*.so"))
    return hits[0] if hits else None


def _stale(target: str) -> bool:
    srcs = glob.glob(os.path.join(HERE, "csrc", "*"))
    return os.path.getmtime(target) < max(os.path.getmtime(p) for p in srcs)


def build(verbose: bool = False) -> str:
    target = built_path()
    if target and not _stale(target):
        return target
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    from torch.utils.cpp_extension import load
    build_dir = os.path.join(HERE, "_build")
    os.makedirs(build_dir, exist_ok=True)
    load(
        name=NAME,
        sources=[os.path.join(HERE, "csrc", s) for s in SOURCES],
        extra_cuda_cflags=NVCC_FLAGS,
        extra_cflags=["-O2", "-std=c++17"],
        build_directory=build_dir,
        with_cuda=True,
        is_python_module=False,
        verbose=verbose,
    )
    dst = os.path.join(HERE, NAME + ".so")
    shutil.copy2(os.path.join(build_dir, NAME + ".so"), dst)
    return dst
