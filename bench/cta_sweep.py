"""How many CTAs does a collective need to hold the NVLink rate?

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29502 bench/cta_sweep.py --bytes 436M --out sweep.jsonl

Times all-gather (push) and reduce-scatter (pull), and with --ops allreduce the two-shot
all-reduce over peer loads and over the switch (multimem), of one total message size on
registered windows for a list of CTA counts, each both on the per-thread load/store
path and on the bulk-copy-engine path (FLAGCX_BULK_COPY / FLAGCX_BULK_REDUCE switched per
row).  Collectives that run beside GEMMs (sharded training) should take the smallest
count that still reaches the plateau: every CTA is an SM the GEMMs do not get.
CUDA events, median of --iters calls with a barrier before each, max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flagcx_b200 import capi  # noqa: E402
from flagcx_b200.utils.dist import init_world, max_over_ranks  # noqa: E402
from flagcx_b200.utils.symm import SymmetricBuffer  # noqa: E402


def parse_size(s: str) -> int:
    mult = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}
    return int(float(s[:-1]) * mult[s[-1].upper()]) if s[-1].upper() in mult else int(s)


def timed(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3)
    ts.sort()
    return max_over_ranks(ts[len(ts) // 2])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--bytes", default="436M", help="total message (all ranks' blocks together)")
    ap.add_argument("--ctas", default="2,4,8,12,16,24,32,48,96")
    ap.add_argument("--iters", type=int, default=7)
    ap.add_argument("--ops", default="allgather,reducescatter",
                    help="also: allreduce (two-shot over peer loads, and the switch-reduced two-shot when the "
                         "communicator has a multicast binding, i.e. under FLAGCX_NVLS_ENABLE=1)")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    w = init_world()
    n, rank = w.world, w.rank
    total = parse_size(args.bytes) // 2 // (n * 64) * (n * 64)  # bf16 elements
    per = total // n
    send = SymmetricBuffer(w.comm, total * 2)
    recv = SymmetricBuffer(w.comm, total * 2)
    src = send.view(torch.bfloat16, total)
    src.normal_()
    dst = recv.view(torch.bfloat16, total)
    rows = []
    if rank == 0:
        print(f"# world {n}  total {total * 2} bytes  per-rank block {per * 2} bytes", flush=True)
        print(f"{'op':>14} {'path':>7} {'ctas':>5} {'us':>9} {'busGB/s':>9}", flush=True)
    ops = args.ops.split(",")
    if "allreduce" in ops:
        algos = [("twoshot", capi.ALGO_TWOSHOT)] + ([("nvls", capi.ALGO_NVLS_TWOSHOT)] if w.comm.has_multicast else [])
        for path, algo in algos:
            for ctas in [int(x) for x in args.ctas.split(",")]:
                fn = lambda: w.comm.all_reduce_fused(src, dst, total, capi.BFLOAT16, capi.SUM, algo=algo, nctas=ctas)
                us = timed(fn, args.iters)
                assert w.comm.async_error() == 0, w.comm.last_error()
                bw = total * 2 / us / 1e3 * 2 * (n - 1) / n
                rows.append({"op": "allreduce", "path": path, "ctas": ctas, "us": us, "busbw": bw, "n_gpus": n, "bytes": total * 2})
                if rank == 0:
                    print(f"{'allreduce':>14} {path:>7} {ctas:>5} {us:>9.1f} {bw:>9.1f}", flush=True)
    for op in [o for o in ops if o in ("allgather", "reducescatter")]:
        for path in ("threads", "engine"):
            os.environ["FLAGCX_BULK_COPY"] = os.environ["FLAGCX_BULK_REDUCE"] = "1" if path == "engine" else "0"
            os.environ["FLAGCX_BULK_COPY_MIN_BYTES"] = "1"
            for ctas in [int(x) for x in args.ctas.split(",")]:
                if op == "allgather":
                    fn = lambda: w.comm.all_gather(src[:per], dst, per, capi.BFLOAT16, algo=capi.ALGO_PUSH, nctas=ctas)
                else:
                    fn = lambda: w.comm.reduce_scatter_fused(src, dst[:per], per, capi.BFLOAT16, capi.SUM,
                                                             algo=capi.ALGO_PULL, nctas=ctas)
                us = timed(fn, args.iters)
                assert w.comm.async_error() == 0, w.comm.last_error()
                bw = total * 2 / us / 1e3 * (n - 1) / n
                rows.append({"op": op, "path": path, "ctas": ctas, "us": us, "busbw": bw, "n_gpus": n, "bytes": total * 2})
                if rank == 0:
                    print(f"{op:>14} {path:>7} {ctas:>5} {us:>9.1f} {bw:>9.1f}", flush=True)
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    torch.cuda.synchronize()
    dist.barrier()
    send.free()
    recv.free()
    w.comm.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
