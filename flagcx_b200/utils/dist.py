"""Process bootstrap for launches under torchrun (one process per GPU).

torch.distributed (gloo for host objects, NCCL for the comparison runs) is the
plumbing; the flagcx communicator is created from a unique id that rank 0
broadcasts through it.  Rendezvous address and ranks come from the usual
RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT variables.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.distributed as dist

from flagcx_b200 import capi


@dataclass
class World:
    rank: int
    world: int
    local_rank: int
    comm: capi.Comm


def env_rank():
    return (int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)),
            int(os.environ.get("LOCAL_RANK", 0)))


def init_torch_dist(backend: str | None = None) -> None:
    rank, world, local = env_rank()
    if dist.is_initialized():
        return
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29577")
    if torch.cuda.is_available():
        torch.cuda.set_device(local)
    if backend is None:
        backend = "cpu:gloo,cuda:nccl" if torch.cuda.is_available() else "gloo"
    dist.init_process_group(backend=backend, rank=rank, world_size=world)


def init_world(backend: str | None = None) -> World:
    """Initialises torch.distributed (if needed) and a flagcx communicator."""
    rank, world, local = env_rank()
    init_torch_dist(backend)
    box = [capi.unique_id_bytes(capi.get_unique_id()) if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    comm = capi.Comm.init_rank(world, capi.unique_id_from_bytes(box[0]), rank)
    return World(rank, world, local, comm)


def max_over_ranks(value: float) -> float:
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
