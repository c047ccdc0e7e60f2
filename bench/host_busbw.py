"""Host-buffer collectives (sockets + shared-memory rings, no GPU) against gloo.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 \
        --master-port 29620 bench/host_busbw.py [--max-bytes 64M] [--out host.jsonl]

Times flagcxAllReduce / AllGather / ReduceScatter / AlltoAll on numpy arrays through the
library's host route (the role of the FlagCX bootstrap adaptor, flagcx/adaptor/ccl/
bootstrap_adaptor.cc in the FlagCX project) and the same operations of torch.distributed's
gloo backend on the same ranks.  Wall-clock per call (these are host operations), a
barrier before each, median of --iters, max over ranks.  Works on a machine without GPUs.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flagcx_b200 import capi  # noqa: E402
from flagcx_b200.utils.dist import init_world, max_over_ranks  # noqa: E402


def parse_size(s: str) -> int:
    mult = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}
    return int(float(s[:-1]) * mult[s[-1].upper()]) if s[-1].upper() in mult else int(s)


def timed(fn, iters, barrier):
    for _ in range(2):
        fn()
    ts = []
    for _ in range(iters):
        barrier()
        t0 = time.perf_counter()
        fn()
        ts.append((time.perf_counter() - t0) * 1e6)
    ts.sort()
    return max_over_ranks(ts[len(ts) // 2])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-bytes", default="1K")
    ap.add_argument("--max-bytes", default="64M")
    ap.add_argument("--iters", type=int, default=9)
    ap.add_argument("--ops", default="allreduce,allgather,reducescatter,alltoall")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    os.environ.setdefault("CUDA_VISIBLE_DEVICES", "")  # host route on any machine
    w = init_world("gloo")
    n, rank = w.world, w.rank
    rows = []
    if rank == 0:
        print(f"# {n} host ranks, float32; microseconds per call (median, max over ranks)")
        print(f"{'op':>14} {'bytes':>10} {'ours us':>10} {'gloo us':>10} {'ratio':>6}", flush=True)
    size = parse_size(args.min_bytes)
    hi = parse_size(args.max_bytes)
    factor = {"allreduce": 2 * (n - 1) / n, "allgather": (n - 1) / n, "reducescatter": (n - 1) / n, "alltoall": (n - 1) / n}
    while size <= hi:
        total = max(size // 4 // n * n, n)  # float32 elements of the whole message
        per = total // n
        rng = np.random.default_rng(rank)
        x = rng.standard_normal(total).astype(np.float32)
        y = np.empty(total, np.float32)
        tx, ty = torch.from_numpy(x.copy()), torch.empty(total)
        for op in args.ops.split(","):
            if op == "allreduce":
                ours = lambda: w.comm.all_reduce(x, y, total, capi.FLOAT, capi.SUM)
                ref = lambda: dist.all_reduce(ty.copy_(tx))
            elif op == "allgather":
                ours = lambda: w.comm.all_gather(x[:per], y, per, capi.FLOAT)
                ref = lambda: dist.all_gather_into_tensor(ty, tx[:per])
            elif op == "reducescatter":
                ours = lambda: w.comm.reduce_scatter(x, y[:per], per, capi.FLOAT, capi.SUM)
                ref = None  # gloo has no reduce-scatter
            else:
                ours = lambda: w.comm.all_to_all(x, y, per, capi.FLOAT)
                ref = lambda: dist.all_to_all_single(ty, tx)
            us = timed(ours, args.iters, w.comm.barrier)
            ref_us = timed(ref, args.iters, dist.barrier) if ref else None
            if op == "allreduce":  # the sum of the seeded inputs, checked once per size
                want = sum(np.random.default_rng(r).standard_normal(total).astype(np.float32).astype(np.float64) for r in range(n))
                ok = bool(np.max(np.abs(y - want) / np.maximum(np.abs(want), 1.0)) < 1e-5)
            else:
                ok = True
            rows.append({"impl": "ours", "op": op, "dtype": "fp32", "bytes": total * 4, "n_gpus": n, "mode": "host",
                         "ours_us": us, "nccl_us": ref_us, "ours_busbw": total * 4 * factor[op] / us / 1e3,
                         "nccl_busbw": (total * 4 * factor[op] / ref_us / 1e3) if ref_us else None, "correct": ok})
            if rank == 0:
                ratio = f"{ref_us / us:.2f}" if ref_us else "-"
                print(f"{op:>14} {total * 4:>10} {us:>10.1f} {(f'{ref_us:.1f}' if ref_us else '-'):>10} {ratio:>6}" + ("" if ok else "  WRONG"), flush=True)
        size *= 4
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    w.comm.barrier()
    w.comm.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
