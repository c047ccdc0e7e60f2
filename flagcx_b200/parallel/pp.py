"""Pipeline parallelism over flagcx send/recv: stage-to-stage activation and gradient
exchange and a 1F1B (one-forward-one-backward) micro-batch schedule.

The FlagCX project offers pipeline stages only ``flagcxSend`` / ``flagcxRecv`` and the
``batch_isend_irecv`` hook of its torch plugin (plugin/torch/flagcx/__init__.py:62-86);
this module is the schedule a framework would put on top.  Each rank owns one stage
(an ``nn.Module``); activations travel forward, their gradients backward, as grouped
send/recv calls on the communicator (NVLink kernels for CUDA tensors, sockets for CPU
tensors).  Shapes are fixed per pipeline, so no shape handshake is needed.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch

from flagcx_b200 import capi

_DT = {torch.float32: capi.FLOAT, torch.bfloat16: capi.BFLOAT16, torch.float16: capi.HALF, torch.float64: capi.DOUBLE}


class PipelineStage:
    """One stage of a linear pipeline: rank r receives from r-1 and sends to r+1."""

    def __init__(self, comm: capi.Comm, module: torch.nn.Module, in_shape: Sequence[int] | None,
                 out_shape: Sequence[int], dtype: torch.dtype = torch.float32, device: str | torch.device = "cpu"):
        self.comm, self.module = comm, module
        self.rank, self.world = comm.rank, comm.nranks
        self.first, self.last = self.rank == 0, self.rank == comm.nranks - 1
        self.in_shape, self.out_shape = (tuple(in_shape) if in_shape is not None else None), tuple(out_shape)
        self.dtype, self.device = dtype, torch.device(device)

    # -- transfers ------------------------------------------------------------------
    def _stream(self):
        """CUDA stages queue their transfers on torch's current stream: the order with the
        stage's compute is the stream's, and the host never waits."""
        return torch.cuda.current_stream(self.device) if self.device.type == "cuda" else None

    def _send(self, t: torch.Tensor, peer: int):
        t = t.contiguous()
        self.comm.send(t, t.numel(), _DT[t.dtype], peer, stream=self._stream())

    def _recv(self, shape, peer: int) -> torch.Tensor:
        t = torch.empty(shape, dtype=self.dtype, device=self.device)
        self.comm.recv(t, t.numel(), _DT[t.dtype], peer, stream=self._stream())
        return t

    def _exchange(self, send: torch.Tensor | None, send_peer: int, recv_shape, recv_peer: int):
        """A send and a receive that may cross: issued as one group so neither blocks the other."""
        out = torch.empty(recv_shape, dtype=self.dtype, device=self.device) if recv_shape is not None else None
        st = self._stream()
        self.comm.group_start()
        if send is not None:
            send = send.contiguous()
            self.comm.send(send, send.numel(), _DT[send.dtype], send_peer, stream=st)
        if out is not None:
            self.comm.recv(out, out.numel(), _DT[out.dtype], recv_peer, stream=st)
        self.comm.group_end()
        return out

    # -- schedule -------------------------------------------------------------------
    def run_1f1b(self, microbatches: Sequence[torch.Tensor] | None, n_micro: int,
                 loss_fn: Callable[[torch.Tensor, int], torch.Tensor] | None = None) -> float:
        """Runs n_micro micro-batches through the pipeline and accumulates parameter
        gradients in ``module`` (call ``optimizer.step()`` afterwards).

        The first stage passes its inputs in ``microbatches``; the last stage passes
        ``loss_fn(output, index) -> scalar`` (already divided by n_micro if a mean over
        micro-batches is wanted).  Returns the summed loss on the last stage, 0 elsewhere.

        Schedule: ``world - rank - 1`` warm-up forwards, then one forward and one
        backward in turn, then the remaining backwards -- at most ``world - rank``
        activations are alive on a stage.
        """
        warmup = min(self.world - self.rank - 1, n_micro)
        steady = n_micro - warmup
        inputs, outputs = [], []
        total = 0.0
        fwd_i = 0

        def forward(x: torch.Tensor | None) -> torch.Tensor:
            nonlocal fwd_i, total
            if self.first:
                x = microbatches[fwd_i].to(self.device)
            else:
                x.requires_grad_(True)
            y = self.module(x)
            if self.last:
                y = loss_fn(y, fwd_i)
                total += float(y.detach())
            inputs.append(x)
            outputs.append(y)
            fwd_i += 1
            return y

        def backward(grad_out: torch.Tensor | None) -> torch.Tensor | None:
            x, y = inputs.pop(0), outputs.pop(0)  # oldest micro-batch in flight
            if self.last:
                y.backward()
            else:
                y.backward(grad_out)
            return None if self.first else x.grad

        prev, nxt = self.rank - 1, self.rank + 1
        # warm-up: fill the pipeline
        for _ in range(warmup):
            y = forward(None if self.first else self._recv(self.in_shape, prev))
            self._send(y.detach(), nxt)  # warmup > 0 implies this is not the last stage
        # steady state: one forward, one backward
        x = None
        if steady > 0 and not self.first:
            x = self._recv(self.in_shape, prev)
        for k in range(steady):
            y = forward(x)
            # the activation goes forward while the gradient of the oldest one comes back
            g = None if self.last else self._exchange(y.detach(), nxt, self.out_shape, nxt)
            gx = backward(g)
            if self.first:
                continue
            if k + 1 < steady:
                # the gradient goes back while the next activation comes in
                x = self._exchange(gx, prev, self.in_shape, prev)
            else:
                self._send(gx, prev)
        # cool-down: drain the backwards of the warm-up micro-batches
        for _ in range(warmup):
            gx = backward(self._recv(self.out_shape, nxt))
            if not self.first:
                self._send(gx, prev)
        return total
