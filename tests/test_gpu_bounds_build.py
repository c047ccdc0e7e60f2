"""The bounds-checking kernel build (make -C csrc bounds): every collective kernel checks the
extent of what it is about to touch against the sizes the host recorded and, on a
violation, reports it and returns without making the access.  It stands in for a memory
checker.  Two runs in child processes that load that build (FLAGCX_LIBRARY): the emulated-
world suite must pass unchanged, and with the host understating every buffer by 16 bytes
(FLAGCX_BOUNDS_TEST_SHRINK) the kernels must report flagcxInvalidArgument instead of
touching memory."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "csrc", "build", "bounds", "libflagcx.so")


def _build():
    subprocess.run(["make", "-C", os.path.join(ROOT, "csrc"), "-j", "16", "bounds"], check=True, capture_output=True)
    return LIB


def test_emulated_world_suite_under_the_bounds_checking_build():
    env = dict(os.environ, FLAGCX_LIBRARY=_build())
    res = subprocess.run([sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", "test_gpu_emu.py"), "-x", "-q",
                          "-k", "allreduce_sum or reduce_scatter_and_allgather or rooted_and_alltoall or pointer_exchange "
                                "or ring_algorithms or small_messages or alltoallv"],
                         cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-2000:]


def test_an_understated_buffer_is_reported_and_not_touched():
    code = r"""
import torch
from flagcx_b200 import capi
n = 4
comms = capi.Comm.emu_world(n, 0)
count = 4096
xs = [torch.ones(count, device="cuda") for _ in range(n)]
outs = [torch.full((count,), -7.0, device="cuda") for _ in range(n)]
for r in range(n):
    comms[r].all_reduce_fused(xs[r], outs[r], count, capi.FLOAT, capi.SUM, algo=capi.ALGO_TWOSHOT)
torch.cuda.synchronize()
codes = [c.async_error() for c in comms]
assert all(code == capi.flagcxInvalidArgument for code in codes), codes
assert "bounds" in comms[0].last_error(), comms[0].last_error()
assert all(bool((o == -7.0).all()) for o in outs), "a kernel wrote although its check failed"
assert float((torch.ones(8, device="cuda") * 2).sum()) == 16.0  # the context is healthy
capi.Comm.emu_world_destroy(comms)
print("ok")
"""
    env = dict(os.environ, FLAGCX_LIBRARY=_build(), FLAGCX_BOUNDS_TEST_SHRINK="16")
    res = subprocess.run([sys.executable, "-c", code], cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "ok" in res.stdout, res.stdout[-2000:] + res.stderr[-3000:]
