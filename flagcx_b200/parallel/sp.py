"""Sequence / context parallelism for attention on top of the collectives:

* Ulysses: an all-to-all turns sequence-sharded activations [S/n, H, D] into head-sharded
  ones [S, H/n, D] before attention and back afterwards (one direct-write all-to-all
  kernel each way on GPUs).
* Ring attention: every rank keeps its query block and passes key/value blocks around
  the ring with grouped send/recv, accumulating softmax online, so no rank ever holds
  the whole sequence.

The FlagCX project supplies only the primitives for these (all-to-all, send/recv); this
module is the thin framework layer over them.  Tensors may live on the GPU (NVLink
kernels) or on the CPU (host path); the math is plain PyTorch.  On the GPU nothing here
blocks the host: collectives are ordered on CUDA streams, and ring attention receives the
next key/value block on a side stream while it computes on the current one.
"""
from __future__ import annotations

import math

import torch

from flagcx_b200 import capi

_DT = {torch.float32: capi.FLOAT, torch.bfloat16: capi.BFLOAT16, torch.float16: capi.HALF, torch.float64: capi.DOUBLE}


def _stream(t: torch.Tensor):
    """The stream a collective on `t` is queued on: torch's current stream (None on the CPU)."""
    return torch.cuda.current_stream(t.device) if t.is_cuda else None


class Ulysses:
    """Head <-> sequence re-sharding by all-to-all (n ranks, H divisible by n)."""

    def __init__(self, comm: capi.Comm):
        self.comm, self.n = comm, comm.nranks

    def seq_to_heads(self, x: torch.Tensor) -> torch.Tensor:
        """[S/n, H, D] on every rank (rank r holds sequence chunk r) -> [S, H/n, D]
        (rank r holds head group r of the whole sequence)."""
        s, H, D = x.shape
        n, h = self.n, H // self.n
        assert h * n == H, "heads must divide by the number of ranks"
        send = x.view(s, n, h, D).permute(1, 0, 2, 3).contiguous()  # block p: head group p of my chunk
        recv = torch.empty_like(send)                                # block q: my head group of chunk q
        self.comm.all_to_all(send, recv, s * h * D, _DT[x.dtype], stream=_stream(x))
        return recv.view(n * s, h, D)

    def heads_to_seq(self, y: torch.Tensor) -> torch.Tensor:
        """Inverse of seq_to_heads: [S, H/n, D] -> [S/n, H, D]."""
        S, h, D = y.shape
        n, s = self.n, S // self.n
        assert s * n == S
        send = y.contiguous().view(n, s, h, D)                       # block p: my heads of chunk p
        recv = torch.empty_like(send)                                # block q: head group q of my chunk
        self.comm.all_to_all(send, recv, s * h * D, _DT[y.dtype], stream=_stream(y))
        return recv.permute(1, 0, 2, 3).reshape(s, n * h, D)


def ring_attention(comm: capi.Comm, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = False) -> torch.Tensor:
    """Attention over a sequence sharded in order across the ranks.  q, k, v: [S/n, H, D]
    (this rank's chunk).  Returns this rank's [S/n, H, D] output.

    n steps: attend to the key/value block currently held while it is already on its way
    to the next rank and the following block is coming in (grouped send/recv on a side
    stream), keeping running maxima and sums in fp32.  With ``causal=True`` blocks from
    later ranks are skipped and the own block is masked.
    """
    n, r = comm.nranks, comm.rank
    s, H, D = q.shape
    scale = 1.0 / math.sqrt(D)
    qf = q.float().permute(1, 0, 2)                          # [H, s, D]
    out = torch.zeros(H, s, D, dtype=torch.float32, device=q.device)
    row_max = torch.full((H, s, 1), -float("inf"), dtype=torch.float32, device=q.device)
    row_sum = torch.zeros(H, s, 1, dtype=torch.float32, device=q.device)
    kv = torch.stack([k, v]).contiguous()                     # travels as one message
    nxt, prv = (r + 1) % n, (r - 1) % n
    cuda = q.is_cuda
    main = torch.cuda.current_stream(q.device) if cuda else None
    side = torch.cuda.Stream(q.device) if cuda and n > 1 else None
    for step in range(n):
        src = (r - step) % n                                  # whose block this is
        incoming, arrived = None, None
        if step + 1 < n and cuda:
            # the exchange of this step runs beside the attention over the block in hand
            incoming = torch.empty_like(kv)
            side.wait_stream(main)                            # kv is complete, `incoming` is allocated
            comm.group_start()
            comm.send(kv, kv.numel(), _DT[kv.dtype], nxt, stream=side)
            comm.recv(incoming, incoming.numel(), _DT[kv.dtype], prv, stream=side)
            comm.group_end()
            arrived = torch.cuda.Event()
            arrived.record(side)
            kv.record_stream(side)
            incoming.record_stream(side)
        if not (causal and src > r):
            kf, vf = kv[0].float().permute(1, 0, 2), kv[1].float().permute(1, 0, 2)
            scores = torch.matmul(qf, kf.transpose(1, 2)) * scale     # [H, s, s]
            if causal and src == r:
                mask = torch.ones(s, s, dtype=torch.bool, device=q.device).tril()
                scores = scores.masked_fill(~mask, -float("inf"))
            blk_max = scores.max(dim=-1, keepdim=True).values
            new_max = torch.maximum(row_max, blk_max)
            p = torch.exp(scores - new_max)
            corr = torch.exp(row_max - new_max)
            out = out * corr + torch.matmul(p, vf)
            row_sum = row_sum * corr + p.sum(dim=-1, keepdim=True)
            row_max = new_max
        if step + 1 < n:
            if cuda:
                main.wait_event(arrived)
            else:
                incoming = torch.empty_like(kv)
                comm.group_start()
                comm.send(kv, kv.numel(), _DT[kv.dtype], nxt)
                comm.recv(incoming, incoming.numel(), _DT[kv.dtype], prv)
                comm.group_end()
            kv = incoming
    return (out / row_sum).permute(1, 0, 2).to(q.dtype)
