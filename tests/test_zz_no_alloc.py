"""The allocation-free RMSNorm backward (flagcxRmsnormBwdNoAlloc) against the regular,
allocating entry point of this package.

The entry point serves callers that cannot allocate device memory (fixed memory
budgets, latency-critical sections, plug-ins that only get raw pointers and a
stream); it keeps its scratch in a fixed array inside the library.  The test calls
it through its exported C symbol, twice in a row with different shapes -- the
second call finds the first call's leftovers in the shared scratch -- and compares
both results with what ``flagcx_b200.ops`` computes for the same inputs.  The file
name keeps it last in collection order.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from flagcx_b200.ops import build_noalloc
    lib = C.CDLL(build_noalloc.build())
    lib.flagcxRmsnormBwdNoAlloc.restype = C.c_int
    lib.flagcxRmsnormBwdNoAlloc.argtypes = [C.c_void_p] * 6 + [C.c_long, C.c_int, C.c_void_p]
    return lib


def _case(lib, rows, hidden, seed):
    from flagcx_b200 import ops
    gen = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, hidden, device="cuda", generator=gen).to(torch.bfloat16)
    g = torch.randn(rows, hidden, device="cuda", generator=gen).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(hidden, device="cuda", generator=gen)).to(torch.bfloat16)
    _, rstd = ops.ext().rmsnorm_fwd(x, w, 1e-5)
    dx_ref, dw_ref = ops.ext().rmsnorm_bwd(g, x, w, rstd)  # the existing entry point
    dx = torch.empty_like(x)
    dw = torch.empty_like(w)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.flagcxRmsnormBwdNoAlloc(g.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                     dw.data_ptr(), rows, hidden, stream)
    assert rc == 0, rc
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    # same arithmetic; the two libraries are compiled with different fast-math settings
    # and group the per-CTA partial sums differently, hence the tolerance the other
    # RMSNorm tests use
    assert (dx.float() - dx_ref.float()).abs().max().item() < 0.05
    err =((dw.float() - dw_ref.float()).abs() / dw_ref.float().abs().clamp(min=1.0)).max().item()
    assert err < 0.05, err


def test_no_alloc_rmsnorm_backward_matches_regular_entry_point_twice():
    lib = _lib()
    _case(lib, rows=300, hidden=4096, seed=1)   # more rows than CTAs: every scratch row is used
    _case(lib, rows=5, hidden=1024, seed=2)     # fewer rows, smaller width: stale scratch must not leak in


def test_no_alloc_rejects_sizes_beyond_its_scratch():
    lib = _lib()
    t = torch.zeros(16, device="cuda", dtype=torch.bfloat16)
    r = torch.zeros(1, device="cuda")
    rc = lib.flagcxRmsnormBwdNoAlloc(t.data_ptr(), t.data_ptr(), t.data_ptr(), r.data_ptr(), t.data_ptr(),
                                     t.data_ptr(), 1, 16384, None)
    assert rc != 0
    rc = lib.flagcxRmsnormBwdNoAlloc(t.data_ptr(), t.data_ptr(), t.data_ptr(), r.data_ptr(), t.data_ptr(),
                                     t.data_ptr(), 1, 12, None)
    assert rc != 0
    torch.cuda.synchronize()
