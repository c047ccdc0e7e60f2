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


def build(verbose: bool = False) -> None:
    build_core(verbose=verbose)
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
