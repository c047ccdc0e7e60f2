"""Compiles the ProcessGroup extension in-tree (flagcx_b200/torch_backend/_C*.so)."""
from __future__ import annotations

import glob
import os
import shutil

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
NAME = "_flagcx_torch_C"


def built_path() -> str | None:
    hits = glob.glob(os.path.join(HERE, NAME + "*.so"))
    return hits[0] if hits else None


def _stale(target: str) -> bool:
    src = os.path.join(HERE, "csrc", "process_group_flagcx.cpp")
    hdrs = glob.glob(os.path.join(ROOT, "csrc", "include", "*.h"))
    newest = max(os.path.getmtime(p) for p in [src] + hdrs)
    return os.path.getmtime(target) < newest


def build(verbose: bool = False) -> str:
    target = built_path()
    if target and not _stale(target):
        return target
    from torch.utils.cpp_extension import load
    from flagcx_b200 import capi
    capi.lib()  # resident (RTLD_GLOBAL) so that the freshly linked extension can be loaded
    build_dir = os.path.join(HERE, "_build")
    os.makedirs(build_dir, exist_ok=True)
    lib_dir = os.path.join(ROOT, "flagcx_b200", "lib")
    load(
        name=NAME,
        sources=[os.path.join(HERE, "csrc", "process_group_flagcx.cpp")],
        extra_include_paths=[os.path.join(ROOT, "csrc", "include"), "/usr/local/cuda/include"],
        extra_cflags=["-O2", "-std=c++17"],
        extra_ldflags=[f"-L{lib_dir}", "-lflagcx", "-L/usr/local/cuda/lib64", "-lcudart"],
        build_directory=build_dir,
        with_cuda=True,
        is_python_module=False,
        verbose=verbose,
    )
    out = os.path.join(build_dir, NAME + ".so")
    dst = os.path.join(HERE, NAME + ".so")
    shutil.copy2(out, dst)
    return dst
