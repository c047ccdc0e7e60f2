"""Tensor parallelism: the tcgen05 GEMM and the two fused layers built on it.

``gemm_bf16``               D = A @ B.T on the 5th-generation tensor cores
``AllGatherGemm``           column-parallel linear: sequence-sharded activations are
                            exchanged over NVLink inside the GEMM kernel
``GemmReduceScatter``       row-parallel linear: partial products are delivered to the
                            owning rank and summed inside the GEMM kernel
"""
from __future__ import annotations

import ctypes as C

import torch

from flagcx_b200 import capi
from flagcx_b200.utils.symm import tensor_from_ptr

MODE_AG_GEMM = 1
MODE_GEMM_RS = 2


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """a: [M, K], b: [N, K] (both bf16, contiguous) -> [M, N] bf16."""
    assert a.dtype == b.dtype == torch.bfloat16 and a.is_contiguous() and b.is_contiguous()
    M, K = a.shape
    N = b.shape[0]
    assert b.shape[1] == K
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    if stream is None:
        stream = torch.cuda.current_stream(a.device)
    capi.check(capi.lib().flagcxGemmBf16(capi._ptr(a), capi._ptr(b), capi._ptr(out), M, N, K,
                                         capi._stream_arg(stream)), "flagcxGemmBf16")
    return out


class _TpGemm:
    def __init__(self, comm: capi.Comm, mode: int, M: int, N: int, K: int):
        self.comm, self.mode, self.M, self.N, self.K = comm, mode, M, N, K
        self.n = comm.nranks
        h = C.c_void_p()
        capi.check(capi.lib().flagcxTpGemmCreate(comm.h, mode, M, N, K, C.byref(h)), "flagcxTpGemmCreate", comm.h)
        self.h = h

    def close(self) -> None:
        if self.h:
            capi.check(capi.lib().flagcxTpGemmDestroy(self.h), "flagcxTpGemmDestroy")
            self.h = None


class AllGatherGemm(_TpGemm):
    """D[M, N] = all_gather(x_shard)[M, K] @ w[N, K].T in one kernel."""

    def __init__(self, comm: capi.Comm, M: int, N: int, K: int, device: int | None = None):
        super().__init__(comm, MODE_AG_GEMM, M, N, K)
        p = C.c_void_p()
        capi.check(capi.lib().flagcxTpGemmGetShard(self.h, C.byref(p)), "flagcxTpGemmGetShard")
        dev = torch.cuda.current_device() if device is None else device
        rows = M // self.n
        self.shard = tensor_from_ptr(p.value, rows * K * 2, dev).view(torch.bfloat16).view(rows, K)

    def __call__(self, w: torch.Tensor, out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
        """The caller has written its activation shard into ``self.shard``."""
        assert w.dtype == torch.bfloat16 and w.is_contiguous() and tuple(w.shape) == (self.N, self.K)
        if out is None:
            out = torch.empty(self.M, self.N, dtype=torch.bfloat16, device=w.device)
        if stream is None:
            stream = torch.cuda.current_stream(w.device)
        capi.check(capi.lib().flagcxTpAllGatherGemm(self.h, capi._ptr(w), capi._ptr(out), capi._stream_arg(stream)),
                   "flagcxTpAllGatherGemm", self.comm.h)
        return out

    def close(self) -> None:
        self.shard = None
        super().close()


class GemmReduceScatter(_TpGemm):
    """out[M/n, N] = reduce_scatter(x[M, K] @ w[N, K].T) in one kernel."""

    def __init__(self, comm: capi.Comm, M: int, N: int, K: int):
        super().__init__(comm, MODE_GEMM_RS, M, N, K)

    def __call__(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
        assert x.dtype == w.dtype == torch.bfloat16 and x.is_contiguous() and w.is_contiguous()
        assert tuple(x.shape) == (self.M, self.K) and tuple(w.shape) == (self.N, self.K)
        if out is None:
            out = torch.empty(self.M // self.n, self.N, dtype=torch.bfloat16, device=x.device)
        if stream is None:
            stream = torch.cuda.current_stream(x.device)
        capi.check(capi.lib().flagcxTpGemmReduceScatter(self.h, capi._ptr(x), capi._ptr(w), capi._ptr(out),
                                                        capi._stream_arg(stream)), "flagcxTpGemmReduceScatter", self.comm.h)
        return out
