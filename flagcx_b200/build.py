"""Builds every native component in-tree: libflagcx.so (make -C csrc), the fused-op
extension and the torch ProcessGroup extension.  Re-running is incremental."""
from __future__ import annotations

import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def build_core(jobs: int | None = None, verbose: bool = False) -> str:
    jobs = jobs or os.cpu_count() or 4
    cmd = ["make", "-C", os.path.join(ROOT, "csrc"), f"-j{jobs}"]
    res = subprocess.run(cmd, capture_output=not verbose, text=True)
    if res.returncode != 0:
        sys.stderr.write((res.stdout or "") + (res.stderr or ""))
        raise RuntimeError("building libflagcx.so failed")
    return os.path.join(ROOT, "flagcx_b200", "lib", "libflagcx.so")


def build_devtest(verbose: bool = False) -> str:
    """The device-API conformance kernels (csrc/tests/device_api_kernels.cu) as a shared
    library next to their source; tests/test_gpu_device_api.py loads it."""
    src = os.path.join(ROOT, "csrc", "tests", "device_api_kernels.cu")
    lib = os.path.join(ROOT, "csrc", "tests", "libflagcx_devtest.so")
    inc = os.path.join(ROOT, "csrc", "include")
    deps = [src] + [os.path.join(inc, f) for f in os.listdir(inc)]
    if os.path.exists(lib) and os.path.getmtime(lib) >= max(os.path.getmtime(d) for d in deps):
        return lib
    cmd = ["/usr/local/cuda/bin/nvcc", "-std=c++17", "-O2", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
           "-shared", "-Xcompiler", "-fPIC", "-cudart", "shared", "-I" + os.path.join(ROOT, "csrc", "include"), src, "-o", lib]
    res = subprocess.run(cmd, capture_output=not verbose, text=True)
    if res.returncode != 0:
        sys.stderr.write((res.stdout or "") + (res.stderr or ""))
        raise RuntimeError("building the device-API test kernels failed")
    return lib


def build_bounds(jobs: int | None = None, verbose: bool = False) -> str:
    """The kernels once more with -DFLAGCX_BOUNDS_CHECK (csrc/build/bounds/libflagcx.so): every
    kernel verifies the extent of its accesses first; tests/test_gpu_bounds_build.py runs
    the emulated-world suite against it."""
    jobs = jobs or os.cpu_count() or 4
    res = subprocess.run(["make", "-C", os.path.join(ROOT, "csrc"), f"-j{jobs}", "bounds"], capture_output=not verbose, text=True)
    if res.returncode != 0:
        sys.stderr.write((res.stdout or "") + (res.stderr or ""))
        raise RuntimeError("building the bounds-checking libflagcx.so failed")
    return os.path.join(ROOT, "csrc", "build", "bounds", "libflagcx.so")


def build(verbose: bool = False) -> None:
    build_core(verbose=verbose)
    build_bounds(verbose=verbose)
    build_devtest(verbose=verbose)
    try:
        from flagcx_b200.torch_backend import build as tb
    except ImportError:
        tb = None
    if tb is not None:
        tb.build(verbose=verbose)
    try:
        from flagcx_b200.ops import build as ob
    except ImportError:
        ob = None
    if ob is not None:
        ob.build(verbose=verbose)
    from flagcx_b200.ops import build_noalloc
    build_noalloc.build(verbose=verbose)


if __name__ == "__main__":
    build(verbose=True)
