"""The allocation-free RMSNorm backward (flagcxRmsnormBwdNoAlloc).

The entry point serves callers that cannot allocate device memory (fixed memory
budgets, latency-critical sections, plug-ins that only get raw pointers and a
stream); it keeps its scratch in a fixed array inside the library.  The test calls
it through its exported C symbol, several times in a row with different shapes -- each
call finds the previous call's leftovers in the shared scratch -- and compares every
result with two oracles: a plain PyTorch fp32 autograd RMSNorm, and the regular,
allocating entry point of this package.  "Allocates nothing" is checked against the
driver's own free-memory figure, which also sees allocations that bypass torch.  The
file name keeps it last in collection order.
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


def _call(lib, g, x, w, rstd, dx, dw, rows, hidden):
    stream = torch.cuda.current_stream().cuda_stream
    return lib.flagcxRmsnormBwdNoAlloc(g.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                       dw.data_ptr(), rows, hidden, stream)


def _case(lib, rows, hidden, seed):
    from flagcx_b200 import ops
    eps = 1e-5
    gen = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, hidden, device="cuda", generator=gen).to(torch.bfloat16)
    g = torch.randn(rows, hidden, device="cuda", generator=gen).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(hidden, device="cuda", generator=gen)).to(torch.bfloat16)
    # oracle 1: the same operation in plain PyTorch fp32 with autograd
    xf, wf = x.float().requires_grad_(), w.float().requires_grad_()
    rstd_ref = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    (xf * rstd_ref * wf).backward(g.float())
    # oracle 2: the existing, allocating entry point
    _, rstd = ops.ext().rmsnorm_fwd(x, w, eps)
    dx_old, dw_old = ops.ext().rmsnorm_bwd(g, x, w, rstd)
    dx = torch.empty_like(x)
    dw = torch.empty_like(w)
    assert _call(lib, g, x, w, rstd, dx, dw, rows, hidden) == 0  # loads the module on first use
    torch.cuda.synchronize()
    dx.zero_()
    dw.zero_()
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    assert _call(lib, g, x, w, rstd, dx, dw, rows, hidden) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after >= free_before, "the call took device memory from the driver"
    assert (dx.float() - xf.grad).abs().max().item() < 0.05
    err = ((dw.float() - wf.grad).abs() / wf.grad.abs().clamp(min=1.0)).max().item()
    assert err < 0.05, err
    # same arithmetic as the regular entry point; the two libraries are compiled with
    # different fast-math settings and group the per-CTA partial sums differently
    assert (dx.float() - dx_old.float()).abs().max().item() < 0.05
    err = ((dw.float() - dw_old.float()).abs() / dw_old.float().abs().clamp(min=1.0)).max().item()
    assert err < 0.05, err


def test_no_alloc_rmsnorm_backward_matches_fp32_autograd_and_regular_entry_point():
    lib = _lib()
    _case(lib, rows=300, hidden=4096, seed=1)   # more rows than CTAs: every scratch row is used
    _case(lib, rows=5, hidden=1024, seed=2)     # fewer rows, smaller width: stale scratch must not leak in
    _case(lib, rows=200, hidden=8192, seed=3)   # the documented maximum: both packs of every thread
    _case(lib, rows=131, hidden=5120, seed=4)   # a partly filled second pack, more rows than CTAs
    _case(lib, rows=3, hidden=8, seed=5)        # one pack in all


def test_no_alloc_zero_rows_gives_a_zero_weight_gradient():
    lib = _lib()
    hidden = 2048
    x = torch.empty(0, hidden, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(hidden, device="cuda", dtype=torch.bfloat16)
    rstd = torch.empty(1, device="cuda")
    dw = torch.full((hidden,), 7.0, device="cuda", dtype=torch.bfloat16)
    dummy = torch.zeros(16, device="cuda", dtype=torch.bfloat16)
    # pointers must be valid and aligned even though no row is read
    rc = lib.flagcxRmsnormBwdNoAlloc(dummy.data_ptr(), dummy.data_ptr(), w.data_ptr(), rstd.data_ptr(), dummy.data_ptr(),
                                     dw.data_ptr(), 0, hidden, None)
    assert rc == 0
    torch.cuda.synchronize()
    assert float(dw.float().abs().max()) == 0.0
    del x


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
