"""Offline tuner: measure (algorithm x CTA count) per operation and message size on this
machine's GPUs and write the table that communicators load through FLAGCX_TUNE_FILE.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29410 -m flagcx_b200.tune --out flagcx_tune.json \
        [--ops allreduce,allgather,reducescatter,alltoall] [--min-bytes 1K] [--max-bytes 256M] [--iters 10]

    FLAGCX_TUNE_FILE=flagcx_tune.json  <any program using the library>

Every candidate is timed with CUDA events on registered scratch buffers, the slowest
rank counts, and a candidate replaces the heuristic choice only when it is more than 5 %
faster (the FlagCX tuner's hysteresis, flagcx/core/flagcx_tuner.cc:297).  Rank 0 writes
the file and prints what changed.
"""
from __future__ import annotations

import argparse
import sys

from flagcx_b200 import capi
from flagcx_b200.utils.dist import init_world

OPS = {"allreduce": capi.OP_ALLREDUCE, "allgather": capi.OP_ALLGATHER, "reducescatter": capi.OP_REDUCESCATTER,
       "alltoall": capi.OP_ALLTOALL}
ALGO_NAMES = ["oneshot", "twoshot", "nvls_oneshot", "nvls_twoshot", "push", "pull", "nvls", "ll", "ring", "copy_engine"]


def parse_size(s: str) -> int:
    s = s.strip().upper()
    mult = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}.get(s[-1], 1)
    return int(float(s[:-1]) * mult) if s[-1] in "KMG" else int(s)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--ops", default="allreduce,allgather,reducescatter,alltoall")
    ap.add_argument("--min-bytes", default="1K")
    ap.add_argument("--max-bytes", default="256M")
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    w = init_world()
    if not w.comm.device_path:
        if w.rank == 0:
            print("flagcx_b200.tune: the ranks do not share an NVLink domain; nothing to tune", file=sys.stderr)
        return 1
    lo, hi = parse_size(args.min_bytes), parse_size(args.max_bytes)
    ops = [o for o in args.ops.split(",") if o]
    before = {}
    for name in ops:
        size = lo
        while size <= hi:
            before[(name, size)] = w.comm.tuner_query(OPS[name], size)
            size *= 2
    for name in ops:
        w.comm.tune(OPS[name], capi.BFLOAT16, lo, hi, args.iters)
    if w.rank == 0:
        w.comm.tuner_save(args.out)
        print(f"{'op':>13} {'bytes':>11}  heuristic -> tuned")
        for (name, size), old in before.items():
            new = w.comm.tuner_query(OPS[name], size)
            mark = "" if tuple(new) == tuple(old) else "   *"
            print(f"{name:>13} {size:>11}  {ALGO_NAMES[old[0]]}/{old[1]} -> {ALGO_NAMES[new[0]]}/{new[1]}{mark}")
        print(f"wrote {args.out}")
        # every stored choice against the fastest candidate measured for its bucket
        import json
        worst = 1.0
        for e in json.load(open(args.out))["entries"]:
            if e.get("best_usec", 0) > 0 and e.get("usec", 0) > 0:
                worst = max(worst, e["usec"] / e["best_usec"])
        print(f"slowest stored choice relative to the best candidate measured for its size: {worst:.3f}x "
              f"({'within' if worst <= 1.0 / 0.95 + 1e-6 else 'NOT within'} the 5 % hysteresis)")
    w.comm.barrier()
    w.comm.destroy()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
