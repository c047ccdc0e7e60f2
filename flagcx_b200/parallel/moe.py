"""Expert parallelism: fused dispatch (all-to-all + permute) and combine (all-to-all +
top-k weighted sum) over NVLink, plus a plain PyTorch reference used by the tests
and as the comparison arm of the MoE benchmark.
"""
from __future__ import annotations

import ctypes as C

import torch

from flagcx_b200 import capi
from flagcx_b200.utils.symm import tensor_from_ptr


class MoeDispatcher:
    """Owns the peer-mapped buffers of one MoE layer.  Creation and destruction are
    collective."""

    def __init__(self, comm: capi.Comm, max_tokens: int, hidden: int, topk: int, n_experts: int,
                 capacity_rows: int, device: int | None = None):
        self.comm = comm
        self.hidden, self.topk, self.n_experts = hidden, topk, n_experts
        self.capacity = capacity_rows
        self.device = torch.cuda.current_device() if device is None else device
        h = C.c_void_p()
        capi.check(capi.lib().flagcxMoeCreate(comm.h, max_tokens, hidden, topk, n_experts, C.c_size_t(capacity_rows),
                                              C.byref(h)), "flagcxMoeCreate", comm.h)
        self.h = h
        recv, out, offs = C.c_void_p(), C.c_void_p(), C.c_void_p()
        capi.check(capi.lib().flagcxMoeGetBuffers(h, C.byref(recv), C.byref(out), C.byref(offs)), "flagcxMoeGetBuffers")
        nbytes = capacity_rows * hidden * 2
        self.recv_rows = tensor_from_ptr(recv.value, nbytes, self.device).view(torch.bfloat16).view(capacity_rows, hidden)
        self.expert_out = tensor_from_ptr(out.value, nbytes, self.device).view(torch.bfloat16).view(capacity_rows, hidden)
        self.epr = n_experts // comm.nranks
        self.expert_offsets = tensor_from_ptr(offs.value, 4 * (self.epr + 1), self.device).view(torch.int32)

    def dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, stream=None) -> None:
        """x: [T, hidden] bf16; topk_idx: [T, topk] int32 (global expert ids)."""
        assert x.dtype == torch.bfloat16 and x.is_contiguous() and topk_idx.dtype == torch.int32 and topk_idx.is_contiguous()
        self._idx = topk_idx  # the combine reads it again
        capi.check(capi.lib().flagcxMoeDispatch(self.h, capi._ptr(x), capi._ptr(topk_idx), x.shape[0],
                                                capi._stream_arg(stream)), "flagcxMoeDispatch", self.comm.h)

    def combine(self, topk_weights: torch.Tensor, out: torch.Tensor, stream=None) -> None:
        """topk_weights: [T, topk] fp32; out: [T, hidden] bf16."""
        assert topk_weights.dtype == torch.float32 and topk_weights.is_contiguous() and out.is_contiguous()
        capi.check(capi.lib().flagcxMoeCombine(self.h, capi._ptr(topk_weights), capi._ptr(out), out.shape[0],
                                               capi._stream_arg(stream)), "flagcxMoeCombine", self.comm.h)

    def close(self) -> None:
        if self.h:
            self.recv_rows = self.expert_out = self.expert_offsets = None
            capi.check(capi.lib().flagcxMoeDestroy(self.h), "flagcxMoeDestroy")
            self.h = None


def route(logits: torch.Tensor, topk: int):
    """Softmax gating over the top-k logits: returns (idx int32 [T,k], weights fp32 [T,k])."""
    vals, idx = logits.float().topk(topk, dim=-1)
    return idx.to(torch.int32).contiguous(), torch.softmax(vals, dim=-1).contiguous()


def reference_moe(xs, idxs, weights, expert_fn, n_experts):
    """Whole-world reference on CPU tensors in fp32: out[r][t] = sum_k w * expert_fn(e, x[r][t])."""
    outs = []
    for x, idx, w in zip(xs, idxs, weights):
        xf = x.float()
        out = torch.zeros_like(xf)
        for k in range(idx.shape[1]):
            e = idx[:, k].long()
            y = torch.stack([expert_fn(int(e[t]), xf[t]) for t in range(x.shape[0])]) if x.shape[0] else xf
            out += w[:, k:k + 1] * y
        outs.append(out)
    return outs
