"""Bus-bandwidth sweep: allreduce / reduce-scatter / all-gather / alltoall, bf16 and
fp32, message sizes in powers of two, this library against NCCL (torch.distributed)
on identical inputs.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N \
        --master-addr 127.0.0.1 --master-port 29501 bench/busbw.py --max-bytes 1G

Timing: CUDA events on the launching stream, one pair per iteration, an L2 flush
(256 MiB write) between iterations, median over iterations, max over ranks.
busBW uses the FlagCX test-suite factors (test/perf/host_api/test_allreduce.cpp:8-18
and test_allgather.cpp:13-15 in the FlagCX project): 2(n-1)/n for allreduce, (n-1)/n
for the others.  Inputs are uniform in [-1, 1) from seed=rank; every size is checked
against the NCCL result before it is timed.
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

DT = {"bf16": (capi.BFLOAT16, torch.bfloat16), "fp32": (capi.FLOAT, torch.float32)}


def parse_size(s: str) -> int:
    mult = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}
    return int(float(s[:-1]) * mult[s[-1].upper()]) if s[-1].upper() in mult else int(s)


def timed(fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.add_(1)
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3)  # us
    times.sort()
    return max_over_ranks(times[len(times) // 2])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ops", default="allreduce,reducescatter,allgather,alltoall")
    ap.add_argument("--dtypes", default="bf16,fp32")
    ap.add_argument("--min-bytes", default="1K")
    ap.add_argument("--max-bytes", default="256M")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--no-nccl", action="store_true")
    ap.add_argument("--staged", action="store_true", help="use plain torch tensors (staged path) instead of registered buffers")
    ap.add_argument("--fused", action="store_true", help="allreduce variant with scale=1/world and bf16->fp32 cast in-kernel")
    ap.add_argument("--tune", action="store_true", help="run the tuner over the sweep range first")
    ap.add_argument("--algo", type=int, default=capi.ALGO_AUTO)
    ap.add_argument("--nctas", type=int, default=0)
    ap.add_argument("--out", default="")
    args = ap.parse_args()

    w = init_world()

    def _abort_on_error(tp, val, tb):
        # leave no memory bound to a multicast object behind when this rank dies of an error
        try:
            w.comm.abort()
        finally:
            sys.__excepthook__(tp, val, tb)

    sys.excepthook = _abort_on_error
    n, rank = w.world, w.rank
    lo, hi = parse_size(args.min_bytes), parse_size(args.max_bytes)
    flush = None if args.no_flush else torch.zeros(64 << 20, dtype=torch.float32, device="cuda")
    sendbuf = SymmetricBuffer(w.comm, hi, register=not args.staged)
    recvbuf = SymmetricBuffer(w.comm, hi * (2 if args.fused else 1), register=not args.staged)
    nccl_send = torch.empty(hi, dtype=torch.uint8, device="cuda")
    nccl_recv = torch.empty(hi * (2 if args.fused else 1), dtype=torch.uint8, device="cuda")
    if args.tune:
        for op in (capi.OP_ALLREDUCE, capi.OP_ALLGATHER, capi.OP_REDUCESCATTER):
            w.comm.tune(op, capi.BFLOAT16, lo, min(hi, 1 << 28), 5)
    rows = []
    if rank == 0:
        print(f"# world {n}  nvls {w.comm.has_multicast}  registered {not args.staged}", flush=True)
        print(f"{'op':>13} {'dtype':>5} {'bytes':>11} {'ours_us':>9} {'ours_busGB/s':>12} {'nccl_us':>9} {'nccl_busGB/s':>12} {'ratio':>6} algo ctas",
              flush=True)
    for opname in args.ops.split(","):
        for dtn in args.dtypes.split(","):
            dt, tdt = DT[dtn]
            es = 2 if dtn == "bf16" else 4
            size = lo
            while size <= hi:
                # `size` is the total message: the per-rank block for AG/RS/A2A is size/n
                total = max(size // es, n) // n * n
                per = total // n
                g = torch.Generator(device="cuda").manual_seed(rank)
                src = sendbuf.view(tdt, total)
                src.copy_((torch.rand(total, generator=g, device="cuda") * 2 - 1).to(tdt))
                ncs = nccl_send.view(tdt)[:total]
                ncs.copy_(src)
                if opname == "allreduce":
                    if args.fused:
                        dst = recvbuf.view(torch.float32, total)
                        ours = lambda: w.comm.all_reduce_fused(src, dst, total, dt, capi.SUM, scale=1.0 / n,
                                                               out_dtype=capi.FLOAT, algo=args.algo, nctas=args.nctas)
                        ncd = nccl_recv.view(torch.float32)[:total]

                        def nccl():
                            tmp = ncs.clone()  # NCCL reduces in place: keep the input intact
                            dist.all_reduce(tmp)
                            ncd.copy_(tmp.float().mul_(1.0 / n))
                    else:
                        dst = recvbuf.view(tdt, total)
                        ours = lambda: w.comm.all_reduce_fused(src, dst, total, dt, capi.SUM, algo=args.algo,
                                                               nctas=args.nctas)
                        ncd = nccl_recv.view(tdt)[:total]

                        def nccl():
                            ncd.copy_(ncs)
                            dist.all_reduce(ncd)
                    factor, opcode = 2 * (n - 1) / n, capi.OP_ALLREDUCE
                elif opname == "reducescatter":
                    dst = recvbuf.view(tdt, per)
                    ours = lambda: w.comm.reduce_scatter(src, dst, per, dt, capi.SUM)
                    ncd = nccl_recv.view(tdt)[:per]
                    nccl = lambda: dist.reduce_scatter_tensor(ncd, ncs)
                    factor, opcode = (n - 1) / n, capi.OP_REDUCESCATTER
                elif opname == "allgather":
                    dst = recvbuf.view(tdt, total)
                    ours = lambda: w.comm.all_gather(src[:per], dst, per, dt, algo=args.algo, nctas=args.nctas)
                    ncd = nccl_recv.view(tdt)[:total]
                    nccl = lambda: dist.all_gather_into_tensor(ncd, ncs[:per])
                    factor, opcode = (n - 1) / n, capi.OP_ALLGATHER
                else:
                    dst = recvbuf.view(tdt, total)
                    ours = lambda: w.comm.all_to_all(src, dst, per, dt)
                    ncd = nccl_recv.view(tdt)[:total]
                    nccl = lambda: dist.all_to_all_single(ncd, ncs)
                    factor, opcode = (n - 1) / n, capi.OP_ALLTOALL
                # correctness against NCCL on the same inputs
                ours()
                ok = True
                if not args.no_nccl:
                    nccl()
                    torch.cuda.synchronize()
                    a, b = dst[:ncd.numel()].float(), ncd.float()
                    tol = (2 ** -6 if dtn == "bf16" else 1e-5) * max(1, n // 2)
                    ok = bool(((a - b).abs() <= tol * b.abs().clamp(min=1)).all())
                torch.cuda.synchronize()
                assert w.comm.async_error() == 0, w.comm.last_error()
                t_ours = timed(ours, args.iters, args.warmup, flush)
                t_nccl = float("nan") if args.no_nccl else timed(nccl, args.iters, args.warmup, flush)
                nbytes = total * es
                st = w.comm.stats(opcode)
                row = {"op": opname + ("_fused" if args.fused and opname == "allreduce" else ""), "dtype": dtn,
                       "bytes": nbytes, "n_gpus": n, "ours_us": t_ours, "nccl_us": t_nccl,
                       "ours_busbw": nbytes / t_ours / 1e3 * factor, "nccl_busbw": nbytes / t_nccl / 1e3 * factor,
                       "algo": st.lastAlgo, "nctas": st.lastCtas, "correct": ok,
                       "registered": not args.staged}
                rows.append(row)
                if rank == 0:
                    print(f"{row['op']:>13} {dtn:>5} {nbytes:>11} {t_ours:>9.1f} {row['ours_busbw']:>12.1f} {t_nccl:>9.1f} "
                          f"{row['nccl_busbw']:>12.1f} {t_nccl / t_ours:>6.2f} {st.lastAlgo:>4} {st.lastCtas:>4}"
                          f"{'' if ok else '  MISMATCH'}", flush=True)
                size *= 2
    if rank == 0 and args.out:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        with open(args.out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    torch.cuda.synchronize()
    dist.barrier()
    sendbuf.free()
    recvbuf.free()
    w.comm.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
