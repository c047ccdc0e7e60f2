"""Fully-sharded data parallelism (ZeRO-3 style) on symmetric memory.

Every unit of the model (embedding, decoder layer, head) keeps only its 1/world
shard of parameters, gradients and optimizer state.  Around a unit's compute the
engine

  * all-gathers the unit's parameters straight into one of two peer-mapped
    buffers: every rank's kernel writes its shard into all peers' buffers over
    NVLink (no staging, no temporary), on a side stream, one unit ahead of the
    compute (forward) and one unit ahead in reverse (backward);
  * reduce-scatters the unit's gradients out of a peer-mapped gradient buffer: each
    rank's kernel pulls its slice from all peers, accumulates in fp32, applies the
    1/world average and writes bf16 once;
  * finally runs a fused AdamW step on each shard.

With world_size == 1 the gather buffers alias the shards and no collective runs.
The engine needs ``flagcx_b200.capi.Comm`` (the communicator of a "flagcx" process
group works: ``flagcx_b200.torch_backend.comm_of``).
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch

from flagcx_b200 import capi, ops
from flagcx_b200.models.llama import Unit, _numel
from flagcx_b200.utils.symm import SymmetricBuffer

_ALIGN = 64  # elements: every shard starts on a 128-byte boundary
# parameters that the model applies through ops.linear (weight gradient written in place)
_LINEAR_WEIGHTS = {"wqkv", "wo", "w13", "w2", "output"}


class ShardedModel:
    def __init__(self, units: List[Unit], comm: Optional[capi.Comm], rank: int = 0, world: int = 1,
                 device: Optional[torch.device] = None, lr: float = 3e-4, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.1, seed: int = 1234, comm_ctas: Optional[int] = None,
                 overlap_optimizer: Optional[bool] = None):
        self.units = units
        self.comm = comm
        self.rank, self.world = rank, world
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.lr, self.betas, self.eps, self.wd = lr, betas, eps, weight_decay
        self.step_count = 0
        self.dtype = torch.bfloat16
        self.comm_launches = 0
        # How the parameter all-gather moves its data: "copy_engine" = DMA copy engines
        # between two one-CTA barrier kernels, which leaves every SM to the GEMMs it runs
        # beside; "push" = the NVLink kernel (comm_ctas CTAs store into the peers' buffers).
        # The gradient reduce-scatter: "copy_engine" = the copy engines deliver every rank's
        # block into the owner's staging area and comm_ctas CTAs add from local memory only;
        # "pull" = comm_ctas CTAs read the peers' buffers over NVLink and add.
        # Measured on two B200s, Llama-3-8B shape, ms per step in one call: kernels 200.9,
        # copy-engine gather 197.1, copy engines for both 196.1 (16 CTAs: 195.0); one GPU 192.
        self.gather_algo = {"push": capi.ALGO_PUSH, "copy_engine": capi.ALGO_COPY_ENGINE}[
            os.environ.get("FLAGCX_FSDP_ALLGATHER", "copy_engine")]
        self.scatter_algo = {"pull": capi.ALGO_PULL, "copy_engine": capi.ALGO_COPY_ENGINE}[
            os.environ.get("FLAGCX_FSDP_REDUCESCATTER", "copy_engine")]
        # CTAs of the collective kernels that run beside the GEMMs (with the copy engines:
        # of the local reduce only); 0 leaves the choice to the communicator's tuner
        default_ctas = "16" if self.scatter_algo == capi.ALGO_COPY_ENGINE else "24"
        self.comm_ctas = comm_ctas if comm_ctas is not None else int(os.environ.get("FLAGCX_FSDP_CTAS", default_ctas))
        # AdamW of a unit runs on its own stream as soon as that unit's gradients are
        # reduced, underneath the backward pass of the units before it (it is bound by
        # memory bandwidth, the backward GEMMs by the tensor cores), instead of after the
        # whole backward pass.  The update touches only this rank's shard, which no kernel
        # of the current step reads any more.  Measured on B200, Llama-3-8B shape: 200.7 ms
        # against 203.1 per step on two GPUs, but 192.3 against 191.3 on one (the power-capped
        # GEMMs lose what the overlap gains), hence on by default only when sharded.
        env = os.environ.get("FLAGCX_FSDP_OVERLAP_OPTIMIZER")
        self.overlap_optimizer = ((env != "0") if env is not None else world > 1) \
            if overlap_optimizer is None else overlap_optimizer
        self._updated = set()
        assert world == 1 or comm is not None, "a communicator is required for world_size > 1"

        self.numel = [sum(_numel(s) for _, s in u.shapes) for u in units]
        quantum = world * _ALIGN
        self.padded = [(n + quantum - 1) // quantum * quantum for n in self.numel]
        self.shard_numel = [p // world for p in self.padded]
        dev = self.device
        self.shard = [torch.empty(n, dtype=self.dtype, device=dev) for n in self.shard_numel]
        self.exp_avg = [torch.zeros(n, dtype=self.dtype, device=dev) for n in self.shard_numel]
        self.exp_avg_sq = [torch.zeros(n, dtype=self.dtype, device=dev) for n in self.shard_numel]
        self.grad_shard = [torch.zeros(n, dtype=self.dtype, device=dev) for n in self.shard_numel]

        max_padded = max(self.padded)
        self.main = torch.cuda.current_stream(dev)
        self.opt_stream = torch.cuda.Stream(dev)
        if world > 1:
            self.comm_stream = torch.cuda.Stream(dev, priority=-1)
            self._sym = [SymmetricBuffer(comm, max_padded * 2) for _ in range(4)]
            self.param_buf = [self._sym[0].view(self.dtype, max_padded), self._sym[1].view(self.dtype, max_padded)]
            self.grad_buf = [self._sym[2].view(self.dtype, max_padded), self._sym[3].view(self.dtype, max_padded)]
        else:
            self.comm_stream = None
            self._sym = []
            self.param_buf = [None, None]
            self.grad_buf = [None, None]
        # what each parameter buffer currently holds, and the events that order its reuse
        self.resident = [-1, -1]
        self.gather_done = [None, None]   # recorded on the comm stream
        self.compute_done = [None, None]  # recorded on the main stream
        self.rs_done = [None, None]
        self._pending_grads = {}
        self._init_parameters(seed)

    # ------------------------------------------------------------------ storage
    def _views(self, flat: torch.Tensor, u: int, requires_grad: bool) -> List[torch.Tensor]:
        out, off = [], 0
        for _, shape in self.units[u].shapes:
            n = _numel(shape)
            t = flat[off:off + n].view(shape)
            if requires_grad:
                t = t.detach().requires_grad_(True)
            out.append(t)
            off += n
        return out

    def _full_flat(self, u: int) -> torch.Tensor:
        """Where unit u's complete parameters live while it computes."""
        if self.world == 1:
            return self.shard[u]
        return self.param_buf[u % 2][: self.padded[u]]

    def _init_parameters(self, seed: int) -> None:
        # Every rank draws the full unit from the same seed and keeps its slice, so the
        # model is identical for every world size.
        gen = torch.Generator(device=self.device)
        for u, unit in enumerate(self.units):
            gen.manual_seed(seed + u)
            full = torch.empty(self.padded[u], dtype=self.dtype, device=self.device) if self.world > 1 else self.shard[u]
            full.zero_()
            off = 0
            for name, shape in unit.shapes:
                n = _numel(shape)
                view = full[off:off + n]
                if "norm" in name:
                    view.fill_(1.0)
                else:
                    view.normal_(0.0, 0.02, generator=gen)
                off += n
            if self.world > 1:
                s = self.shard_numel[u]
                self.shard[u].copy_(full[self.rank * s:(self.rank + 1) * s])
                del full
        torch.cuda.synchronize(self.device)

    def full_parameters(self) -> List[List[torch.Tensor]]:
        """Gathers every unit (for tests and checkpoints); returns copies."""
        out = []
        for u in range(len(self.units)):
            if self.world == 1:
                flat = self.shard[u].clone()
            else:
                torch.cuda.synchronize(self.device)
                self.comm.all_gather(self.shard[u], self.param_buf[u % 2], self.shard_numel[u], capi.BFLOAT16,
                                     stream=self.main)
                self.resident[u % 2] = -1
                torch.cuda.synchronize(self.device)
                flat = self.param_buf[u % 2][: self.padded[u]].clone()
            out.append(self._views(flat, u, False))
        return out

    def state_dict(self) -> dict:
        """This rank's shards and optimizer state (torch.save-able)."""
        return {"step": self.step_count, "rank": self.rank, "world": self.world,
                "shard": [t.cpu() for t in self.shard], "exp_avg": [t.cpu() for t in self.exp_avg],
                "exp_avg_sq": [t.cpu() for t in self.exp_avg_sq]}

    def load_state_dict(self, sd: dict) -> None:
        assert sd["world"] == self.world and sd["rank"] == self.rank, "checkpoint was written for another sharding"
        self.step_count = sd["step"]
        for dst, src in ((self.shard, sd["shard"]), (self.exp_avg, sd["exp_avg"]), (self.exp_avg_sq, sd["exp_avg_sq"])):
            for d, s in zip(dst, src):
                d.copy_(s)
        self.resident = [-1, -1]

    # ------------------------------------------------------------------ gathers
    def _launch_gather(self, u: int) -> None:
        if self.world == 1 or u < 0 or u >= len(self.units):
            return
        b = u % 2
        if self.resident[b] == u:
            return
        cs = self.comm_stream
        if self.compute_done[b] is not None:
            cs.wait_event(self.compute_done[b])  # previous occupant is no longer needed
        self.comm.all_gather(self.shard[u], self.param_buf[b], self.shard_numel[u], capi.BFLOAT16, stream=cs,
                             algo=self.gather_algo, nctas=self.comm_ctas)
        self.comm_launches += 1
        ev = torch.cuda.Event()
        ev.record(cs)
        self.gather_done[b] = ev
        self.resident[b] = u

    def _acquire(self, u: int, prefetch: int) -> List[torch.Tensor]:
        if self.world > 1:
            self._launch_gather(u)
            self.main.wait_event(self.gather_done[u % 2])
            self._launch_gather(prefetch)
        return self._views(self._full_flat(u), u, True)

    def _release(self, u: int) -> None:
        if self.world > 1:
            ev = torch.cuda.Event()
            ev.record(self.main)
            self.compute_done[u % 2] = ev

    # ------------------------------------------------------------------ gradients
    def _grad_flat(self, u: int) -> torch.Tensor:
        return self.grad_shard[u] if self.world == 1 else self.grad_buf[u % 2]

    def _buffer_free_for(self, u: int) -> None:
        """Before the first gradient of unit u is written: the reduce-scatter that last
        read this gradient buffer must have finished."""
        st = self._pending_grads[u]
        if not st["claimed"]:
            st["claimed"] = True
            if self.world > 1 and self.rs_done[u % 2] is not None:
                self.main.wait_event(self.rs_done[u % 2])

    def _on_grad(self, u: int, k: int, leaf: torch.Tensor) -> None:
        """post-accumulate hook of parameter k of unit u (parameters whose gradient autograd
        materialises itself: norms, embedding): move the gradient into the flat gradient
        buffer; when the unit is complete, reduce-scatter it."""
        self._buffer_free_for(u)
        st = self._pending_grads[u]
        off, n = st["offsets"][k]
        self._grad_flat(u)[off:off + n].copy_(leaf.grad.reshape(-1))
        leaf.grad = None
        self._grad_arrived(u)

    def _grad_arrived(self, u: int) -> None:
        st = self._pending_grads[u]
        st["left"] -= 1
        if st["left"] == 0:
            self._reduce_unit(u)
            del self._pending_grads[u]
            if self.overlap_optimizer:
                self._update_unit_early(u)

    def _update_unit_early(self, u: int) -> None:
        """AdamW of unit u on the optimizer stream, right behind its reduce-scatter (or, on
        one GPU, behind the last kernel of its backward pass)."""
        ss = self.opt_stream
        if self.world == 1:
            ev = torch.cuda.Event()
            ev.record(self.main)
            ss.wait_event(ev)  # gradients complete, and the weights are no longer read
        else:
            ss.wait_event(self.rs_done[u % 2])  # this unit's reduce-scatter, just queued
        b1, b2 = self.betas
        with torch.cuda.stream(ss):
            ops.adamw_flat_(self.shard[u], self.grad_shard[u], self.exp_avg[u], self.exp_avg_sq[u], self.lr, b1, b2,
                            self.eps, self.wd, self.step_count + 1)
        self._updated.add(u)

    def _reduce_unit(self, u: int) -> None:
        if self.world == 1:
            return
        b = u % 2
        pad = self.padded[u] - self.numel[u]
        if pad:
            self.grad_buf[b][self.numel[u]:self.padded[u]].zero_()
        ev = torch.cuda.Event()
        ev.record(self.main)
        cs = self.comm_stream
        cs.wait_event(ev)
        self.comm.reduce_scatter_fused(self.grad_buf[b], self.grad_shard[u], self.shard_numel[u], capi.BFLOAT16, capi.AVG,
                                       algo=self.scatter_algo, nctas=self.comm_ctas, stream=cs)
        self.comm_launches += 1
        done = torch.cuda.Event()
        done.record(cs)
        self.rs_done[b] = done

    def _hook_params(self, u: int, leaves: List[torch.Tensor]) -> None:
        offsets, off = [], 0
        for _, shape in self.units[u].shapes:
            n = _numel(shape)
            offsets.append((off, n))
            off += n
        self._pending_grads[u] = {"left": len(leaves), "offsets": offsets, "claimed": False}
        flat = self._grad_flat(u)
        for k, leaf in enumerate(leaves):
            name, shape = self.units[u].shapes[k]
            if len(shape) == 2 and name in _LINEAR_WEIGHTS:
                # the weight-gradient GEMM writes straight into the flat gradient buffer
                # (ops.linear): no per-parameter gradient tensor, no copy
                off, n = offsets[k]
                leaf._grad_sink = (flat[off:off + n].view(shape), lambda u=u: self._grad_arrived(u))
            else:
                leaf.register_post_accumulate_grad_hook(lambda t, u=u, k=k: self._on_grad(u, k, t))

    # ------------------------------------------------------------------ training step
    def forward_backward(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        last = len(self.units) - 1
        x = tokens
        loss = None
        for u, unit in enumerate(self.units):
            leaves = self._acquire(u, prefetch=u + 1)
            self._hook_params(u, leaves)
            if u == last:
                loss = unit.fn(leaves, x, targets)
            else:
                x = unit.fn(leaves, x)
                if u > 0 or x.requires_grad:
                    # fires when d(loss)/dx is known, i.e. just before unit u runs backward:
                    # make sure its parameters are back and fetch the unit before it
                    x.register_hook(lambda g, u=u: self._pre_backward(u))
            if u != last:
                self._release(u)
        self._buffer_free_for(last)  # the head is the first unit to write gradients
        loss.backward()
        if self.world > 1:
            for ev in self.rs_done:
                if ev is not None:
                    self.main.wait_event(ev)
        return loss.detach()

    def _pre_backward(self, u: int) -> None:
        # unit u's backward is about to be queued and will write into its gradient buffer
        self._buffer_free_for(u)
        if self.world > 1:
            # d(loss)/d(output of u) exists, so all of unit u+1's backward is queued:
            # its parameter buffer may be overwritten by the prefetch below
            self._release(u + 1)
            self._launch_gather(u)
            self.main.wait_event(self.gather_done[u % 2])
            self._launch_gather(u - 1)
        return None

    def optimizer_step(self) -> None:
        self.step_count += 1
        b1, b2 = self.betas
        if self._updated:
            done = torch.cuda.Event()
            done.record(self.opt_stream)
            self.main.wait_event(done)  # the early updates are part of this step
        for u in range(len(self.units)):
            if u in self._updated:
                continue
            ops.adamw_flat_(self.shard[u], self.grad_shard[u], self.exp_avg[u], self.exp_avg_sq[u], self.lr, b1, b2,
                            self.eps, self.wd, self.step_count)
        self._updated.clear()
        if self.world > 1:
            # shards changed: whatever the gather buffers hold is stale
            ev = torch.cuda.Event()
            ev.record(self.main)
            self.compute_done = [ev, ev]
            self.resident = [-1, -1]

    def train_step(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        loss = self.forward_backward(tokens, targets)
        self.optimizer_step()
        return loss

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        self.param_buf = [None, None]
        self.grad_buf = [None, None]
        for s in self._sym:
            s.free()
        self._sym = []


class Trainer:
    """The user-facing loop body: takes a batch from pinned host memory, runs one
    sharded training step and returns the loss as a Python float."""

    def __init__(self, model: ShardedModel):
        self.model = model
        self.device = model.device
        self._tok = None

    def step(self, host_tokens: torch.Tensor) -> float:
        """host_tokens: int64 [seq_len + 1] in pinned memory; inputs are [:-1], targets [1:]."""
        if self._tok is None or self._tok.numel() != host_tokens.numel():
            self._tok = torch.empty(host_tokens.numel(), dtype=torch.long, device=self.device)
        self._tok.copy_(host_tokens, non_blocking=True)
        loss = self.model.train_step(self._tok[:-1], self._tok[1:])
        return float(loss.item())
