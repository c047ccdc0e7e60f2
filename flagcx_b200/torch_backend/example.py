"""Walk through the ``"flagcx"`` torch.distributed backend, one call of each kind.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29400 -m flagcx_b200.torch_backend.example [--cpu]

With GPUs every rank takes ``cuda:LOCAL_RANK`` and the collectives run as NVLink
kernels; with ``--cpu`` (or no GPU) the same calls run over the socket path.  Same
role as plugin/torch/example/example.py in the FlagCX project.
"""
from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist

import flagcx_b200.torch_backend as fcx_torch  # registers backend "flagcx"
from flagcx_b200 import capi


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cpu", action="store_true", help="host tensors over sockets even if GPUs are present")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    use_cuda = torch.cuda.is_available() and not args.cpu
    if use_cuda:
        torch.cuda.set_device(local)
    dev = torch.device("cuda", local) if use_cuda else torch.device("cpu")
    dist.init_process_group("flagcx", rank=rank, world_size=world)

    def say(what, ok):
        if rank == 0:
            print(f"{what:<28} {'ok' if ok else 'MISMATCH'}", flush=True)
        return ok

    good = True
    x = torch.full((1 << 16,), float(rank + 1), device=dev)
    dist.all_reduce(x)
    good &= say("all_reduce(sum)", bool(torch.all(x == world * (world + 1) / 2)))

    x = torch.full((1 << 16,), float(rank + 1), device=dev)
    dist.all_reduce(x, op=dist.ReduceOp.AVG)
    good &= say("all_reduce(avg)", bool(torch.allclose(x, torch.full_like(x, (world + 1) / 2))))

    b = torch.full((256,), float(rank), device=dev)
    dist.broadcast(b, src=world - 1)
    good &= say("broadcast", bool(torch.all(b == world - 1)))

    flat = torch.empty(128 * world, device=dev)
    dist.all_gather_into_tensor(flat, torch.full((128,), float(rank), device=dev))
    good &= say("all_gather_into_tensor", bool(torch.equal(flat, torch.arange(world, device=dev).repeat_interleave(128).float())))

    rs = torch.empty(64, device=dev)
    dist.reduce_scatter_tensor(rs, torch.arange(64 * world, device=dev).float())
    good &= say("reduce_scatter_tensor", bool(torch.equal(rs, torch.arange(64 * rank, 64 * rank + 64, device=dev).float() * world)))

    src = torch.arange(8 * world, device=dev).float() + 100 * rank
    dst = torch.empty(8 * world, device=dev)
    dist.all_to_all_single(dst, src)
    want = torch.cat([torch.arange(8 * rank, 8 * rank + 8, device=dev).float() + 100 * p for p in range(world)])
    good &= say("all_to_all_single", bool(torch.equal(dst, want)))

    # ring exchange: the two calls are coalesced into one grouped launch
    send = torch.full((4096,), float(rank), device=dev)
    recv = torch.empty(4096, device=dev)
    ops = [dist.P2POp(dist.isend, send, (rank + 1) % world), dist.P2POp(dist.irecv, recv, (rank - 1) % world)]
    for w in dist.batch_isend_irecv(ops):
        w.wait()
    good &= say("batch_isend_irecv", bool(torch.all(recv == (rank - 1) % world)))

    dist.barrier()
    say("barrier", True)

    # The communicator behind the group, for what torch.distributed has no name for:
    # here an all-reduce with the 1/world scale and the bf16 -> fp32 conversion fused in.
    if use_cuda:
        comm = fcx_torch.comm_of()
        g = torch.full((1 << 20,), float(rank + 1), device=dev, dtype=torch.bfloat16)
        out = torch.empty(1 << 20, device=dev, dtype=torch.float32)
        comm.all_reduce_fused(g, out, g.numel(), capi.BFLOAT16, capi.SUM, scale=1.0 / world, out_dtype=capi.FLOAT)
        torch.cuda.synchronize()
        good &= say("fused all-reduce (C API)", bool(torch.allclose(out, torch.full_like(out, (world + 1) / 2))))

    dist.destroy_process_group()
    return 0 if good else 1


if __name__ == "__main__":
    raise SystemExit(main())
