"""Bus-bandwidth and latency sweep of every collective, bf16 and fp32, message sizes in
powers of two.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29501 bench/busbw.py --max-bytes 1G --out table.jsonl

Arms (``--impl``):

  ours       this library through its C API (ctypes), on registered windows or, with
             ``--plain``, on ordinary torch tensors; NCCL (torch.distributed) is timed in
             the same process on identical inputs and every size is checked against it.
  ours_pg    the same operations issued through torch.distributed with this library's
             "flagcx" backend (ordinary torch tensors).
  nccl       torch.distributed over NCCL alone.
  reference  torch.distributed over the UNMODIFIED FlagCX torch plugin installed under
             ``--ref-dir`` (default baseline/_ref); with FLAGCX_CUSTOM_OP_ENABLE=1 and an
             install built with COMPILE_KERNEL=1 its own all-reduce kernels serve <= 8 MB.

Timing.  ``--mode bandwidth``: CUDA events on the launching stream, one pair per call,
inputs refilled and an L2 flush (256 MiB write) between calls and outside the events, a
barrier before each call, median over calls, max over ranks.  ``--mode latency``: 100
calls back to back between ONE pair of events, no barrier or flush inside, microseconds
per call, median of 5 repetitions, max over ranks.  Nothing but the collective itself is
inside a timed region of any arm.  busBW uses the FlagCX test-suite factors
(test/perf/host_api/test_allreduce.cpp:8-18, test_allgather.cpp:13-15 in the FlagCX
project): 2(n-1)/n for all-reduce, (n-1)/n for reduce-scatter, all-gather and all-to-all,
1 for the rooted and point-to-point operations.  Inputs are uniform in [-1, 1) from
seed=rank.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

ALL_OPS = ["allreduce", "reducescatter", "allgather", "alltoall", "broadcast", "reduce", "gather", "scatter",
           "alltoallv", "sendrecv", "putsignal"]


def parse_size(s: str) -> int:
    mult = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}
    return int(float(s[:-1]) * mult[s[-1].upper()]) if s[-1].upper() in mult else int(s)


class Timer:
    def __init__(self, args, max_over_ranks, barrier):
        self.args, self.max_over_ranks, self.barrier = args, max_over_ranks, barrier
        self.flush = None if args.no_flush else torch.zeros(64 << 20, dtype=torch.float32, device="cuda")

    def bandwidth(self, fn, prep=None):
        a = self.args
        for _ in range(a.warmup):
            if prep:
                prep()
            fn()
        torch.cuda.synchronize()
        times = []
        for _ in range(a.iters):
            if prep:
                prep()
            if self.flush is not None:
                self.flush.add_(1)
            self.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            times.append(e0.elapsed_time(e1) * 1e3)  # us
        times.sort()
        return self.max_over_ranks(times[len(times) // 2])

    def latency(self, fn, prep=None, calls=100, reps=5):
        if prep:
            prep()
        for _ in range(10):
            fn()
        torch.cuda.synchronize()
        per_call = []
        for _ in range(reps):
            self.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(calls):
                fn()
            e1.record()
            e1.synchronize()
            per_call.append(e0.elapsed_time(e1) * 1e3 / calls)
        per_call.sort()
        return self.max_over_ranks(per_call[len(per_call) // 2])

    def run(self, fn, prep=None):
        return self.latency(fn, prep) if self.args.mode == "latency" else self.bandwidth(fn, prep)


def factor_of(op: str, n: int) -> float:
    if op.startswith("allreduce"):
        return 2 * (n - 1) / n
    if op in ("reducescatter", "allgather", "alltoall", "alltoallv"):
        return (n - 1) / n
    return 1.0


def uneven_counts(per: int, n: int):
    """counts[r][p]: elements rank r sends to rank p; sums to about per*n per rank."""
    return [[max(1, per * (1 + (r + 2 * p) % 3) // 2) for p in range(n)] for r in range(n)]


# ------------------------------------------------------------------------------------------
# torch.distributed arms (ours_pg, nccl, reference)
# ------------------------------------------------------------------------------------------
def pg_ops(opname, n, rank, src, dst, per, total, tdt):
    """(callable, prep, bytes moved per rank as the table's size column) for dist.*"""
    if opname == "allreduce":
        work = dst[:total]
        return (lambda: dist.all_reduce(work)), (lambda: work.copy_(src[:total])), total
    if opname == "reducescatter":
        return (lambda: dist.reduce_scatter_tensor(dst[:per], src[:total])), None, total
    if opname == "allgather":
        return (lambda: dist.all_gather_into_tensor(dst[:total], src[:per])), None, total
    if opname == "alltoall":
        return (lambda: dist.all_to_all_single(dst[:total], src[:total])), None, total
    if opname == "broadcast":
        work = dst[:total]
        return (lambda: dist.broadcast(work, src=0)), (lambda: work.copy_(src[:total])), total
    if opname == "reduce":
        work = dst[:total]
        return (lambda: dist.reduce(work, dst=0)), (lambda: work.copy_(src[:total])), total
    if opname == "gather":
        outs = [dst[p * per:(p + 1) * per] for p in range(n)] if rank == 0 else None
        return (lambda: dist.gather(src[:per], outs, dst=0)), None, total
    if opname == "scatter":
        ins = [src[p * per:(p + 1) * per] for p in range(n)] if rank == 0 else None
        return (lambda: dist.scatter(dst[:per], ins, src=0)), None, total
    if opname == "alltoallv":
        counts = uneven_counts(max(per // 2, 1), n)
        ins = counts[rank]
        outs = [counts[p][rank] for p in range(n)]
        return (lambda: dist.all_to_all_single(dst[:sum(outs)], src[:sum(ins)], outs, ins)), None, sum(ins)
    if opname == "sendrecv":
        def ring():
            ops = [dist.P2POp(dist.isend, src[:total], (rank + 1) % n), dist.P2POp(dist.irecv, dst[:total], (rank - 1) % n)]
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        return ring, None, total
    return None, None, 0


def run_pg_arm(args):
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29577")
    if args.impl == "reference":
        ref_dir = os.path.join(ROOT, args.ref_dir)
        if not os.path.isdir(os.path.join(ref_dir, "flagcx")):
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": f"{args.ref_dir} holds no installed reference package"}))
            return
        sys.path.insert(0, ref_dir)
        os.environ.setdefault("TORCH_DEVICE_BACKEND_AUTOLOAD", "0")
        import flagcx  # noqa: F401  the reference's package registers backend "flagcx"
        if hasattr(flagcx, "init"):
            flagcx.init()
        backend = "flagcx"
    elif args.impl == "ours_pg":
        import flagcx_b200.torch_backend  # noqa: F401
        backend = "flagcx"
    else:
        backend = "nccl"
    dist.init_process_group(backend, rank=rank, world_size=world)
    n = world

    def max_over_ranks(x):
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def barrier():
        dist.barrier()

    timer = Timer(args, max_over_ranks, barrier)
    lo, hi = parse_size(args.min_bytes), parse_size(args.max_bytes)
    sendb = torch.empty(hi * 2, dtype=torch.uint8, device="cuda")
    recvb = torch.empty(hi * 2, dtype=torch.uint8, device="cuda")
    rows = []
    if rank == 0:
        print(f"# impl {args.impl}  world {n}  mode {args.mode}  custom_op {os.environ.get('FLAGCX_CUSTOM_OP_ENABLE', '0')}", flush=True)
        print(f"{'op':>13} {'dtype':>5} {'bytes':>11} {'us':>10} {'busGB/s':>9}", flush=True)
    for opname in args.ops.split(","):
        if opname == "putsignal":
            continue  # one-sided: C API only
        for dtn in args.dtypes.split(","):
            tdt = torch.bfloat16 if dtn == "bf16" else torch.float32
            es = 2 if dtn == "bf16" else 4
            size = lo
            while size <= hi:
                total = max(size // es, n) // n * n
                per = total // n
                g = torch.Generator(device="cuda").manual_seed(rank)
                src = sendb.view(tdt)
                src[:total].copy_((torch.rand(total, generator=g, device="cuda") * 2 - 1).to(tdt))
                dst = recvb.view(tdt)
                fn, prep, moved = pg_ops(opname, n, rank, src, dst, per, total, tdt)
                if fn is None:
                    break
                try:
                    us = timer.run(fn, prep)
                except Exception as e:  # noqa: BLE001  an arm that cannot run an operation says so and goes on
                    if rank == 0:
                        print(f"{opname:>13} {dtn:>5} {total * es:>11}  failed: {e!r}"[:200], flush=True)
                    break
                nbytes = moved * es
                row = {"impl": args.impl, "op": opname, "dtype": dtn, "bytes": nbytes, "n_gpus": n, "mode": args.mode,
                       "us": us, "busbw": nbytes / us / 1e3 * factor_of(opname, n),
                       "custom_op": os.environ.get("FLAGCX_CUSTOM_OP_ENABLE", "0")}
                rows.append(row)
                if rank == 0:
                    print(f"{opname:>13} {dtn:>5} {nbytes:>11} {us:>10.1f} {row['busbw']:>9.1f}", flush=True)
                size *= 2
    if rank == 0 and args.out:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        with open(args.out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


# ------------------------------------------------------------------------------------------
# this library through its C API, NCCL beside it
# ------------------------------------------------------------------------------------------
def run_capi_arm(args):
    from flagcx_b200 import capi
    from flagcx_b200.utils.dist import init_world, max_over_ranks
    from flagcx_b200.utils.symm import SymmetricBuffer

    DT = {"bf16": (capi.BFLOAT16, torch.bfloat16), "fp32": (capi.FLOAT, torch.float32)}
    w = init_world()

    def _abort_on_error(tp, val, tb):
        # leave no memory bound to a multicast object behind when this rank dies of an error
        try:
            w.comm.abort()
        finally:
            sys.__excepthook__(tp, val, tb)

    sys.excepthook = _abort_on_error
    n, rank = w.world, w.rank
    timer = Timer(args, max_over_ranks, dist.barrier)
    lo, hi = parse_size(args.min_bytes), parse_size(args.max_bytes)
    plain = args.plain
    if plain:
        # torch tensors handed to the C API: let the library hear about freed segments, which
        # also makes it export allocations on first use (what the torch backend does itself)
        import flagcx_b200.torch_backend as tb
        tb.follow_torch_allocator(w.comm)
    sendbuf = SymmetricBuffer(w.comm, hi * 2, register=not plain) if not plain else None
    recvbuf = SymmetricBuffer(w.comm, hi * 2, register=not plain) if not plain else None
    plain_send = torch.empty(hi * 2, dtype=torch.uint8, device="cuda") if plain else None
    plain_recv = torch.empty(hi * 2, dtype=torch.uint8, device="cuda") if plain else None
    nccl_send = torch.empty(hi * 2, dtype=torch.uint8, device="cuda")
    nccl_recv = torch.empty(hi * 2, dtype=torch.uint8, device="cuda")
    nccl_tmp = torch.empty(hi, dtype=torch.uint8, device="cuda")
    put_win = None
    if args.tune:
        for op in (capi.OP_ALLREDUCE, capi.OP_ALLGATHER, capi.OP_REDUCESCATTER):
            w.comm.tune(op, capi.BFLOAT16, lo, min(hi, 1 << 28), 5)
    rows = []
    if rank == 0:
        print(f"# impl ours  world {n}  mode {args.mode}  nvls {w.comm.has_multicast}  registered {not plain}  "
              f"user-buffer export {bool(w.comm.user_buffer_stats().enabled)}", flush=True)
        print(f"{'op':>13} {'dtype':>5} {'bytes':>11} {'ours_us':>9} {'ours_busGB/s':>12} {'nccl_us':>9} {'nccl_busGB/s':>12} {'ratio':>6} algo ctas",
              flush=True)

    def view(buf, plainbuf, tdt, numel):
        return plainbuf.view(tdt)[:numel] if plain else buf.view(tdt, numel)

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
                src = view(sendbuf, plain_send, tdt, total)
                src.copy_((torch.rand(total, generator=g, device="cuda") * 2 - 1).to(tdt))
                ncs = nccl_send.view(tdt)[:total]
                ncs.copy_(src)
                nccl = nccl_prep = ours_prep = None
                moved = total
                opcode = capi.OP_ALLREDUCE
                check_numel = total
                if opname == "allreduce":
                    if args.fused:
                        dst = view(recvbuf, plain_recv, torch.float32, total)
                        ours = lambda: w.comm.all_reduce_fused(src, dst, total, dt, capi.SUM, scale=1.0 / n,
                                                               out_dtype=capi.FLOAT, algo=args.algo, nctas=args.nctas)
                        ncd = nccl_recv.view(torch.float32)[:total]
                        tmp = nccl_tmp.view(tdt)[:total]
                        nccl_prep = lambda: tmp.copy_(ncs)  # NCCL reduces in place: refill outside the events

                        def nccl():  # the leanest equivalent: average inside NCCL, one cast kernel
                            dist.all_reduce(tmp, op=dist.ReduceOp.AVG)
                            ncd.copy_(tmp)
                    else:
                        dst = view(recvbuf, plain_recv, tdt, total)
                        ours = lambda: w.comm.all_reduce_fused(src, dst, total, dt, capi.SUM, algo=args.algo,
                                                               nctas=args.nctas)
                        ncd = nccl_recv.view(tdt)[:total]
                        nccl_prep = lambda: ncd.copy_(ncs)
                        nccl = lambda: dist.all_reduce(ncd)
                elif opname == "reducescatter":
                    dst = view(recvbuf, plain_recv, tdt, per)
                    ours = lambda: w.comm.reduce_scatter(src, dst, per, dt, capi.SUM)
                    ncd = nccl_recv.view(tdt)[:per]
                    nccl = lambda: dist.reduce_scatter_tensor(ncd, ncs)
                    opcode, check_numel = capi.OP_REDUCESCATTER, per
                elif opname == "allgather":
                    dst = view(recvbuf, plain_recv, tdt, total)
                    ours = lambda: w.comm.all_gather(src[:per], dst, per, dt, algo=args.algo, nctas=args.nctas)
                    ncd = nccl_recv.view(tdt)[:total]
                    nccl = lambda: dist.all_gather_into_tensor(ncd, ncs[:per])
                    opcode = capi.OP_ALLGATHER
                elif opname == "alltoall":
                    dst = view(recvbuf, plain_recv, tdt, total)
                    ours = lambda: w.comm.all_to_all(src, dst, per, dt)
                    ncd = nccl_recv.view(tdt)[:total]
                    nccl = lambda: dist.all_to_all_single(ncd, ncs)
                    opcode = capi.OP_ALLTOALL
                elif opname == "broadcast":
                    dst = view(recvbuf, plain_recv, tdt, total)
                    ours_prep = lambda: dst.copy_(src)
                    ours = lambda: w.comm.broadcast(dst, dst, total, dt, 0)
                    ncd = nccl_recv.view(tdt)[:total]
                    nccl_prep = lambda: ncd.copy_(ncs)
                    nccl = lambda: dist.broadcast(ncd, src=0)
                    opcode = capi.OP_BROADCAST
                elif opname == "reduce":
                    dst = view(recvbuf, plain_recv, tdt, total)
                    ours = lambda: w.comm.reduce(src, dst, total, dt, capi.SUM, 0)
                    ncd = nccl_recv.view(tdt)[:total]
                    nccl_prep = lambda: ncd.copy_(ncs)
                    nccl = lambda: dist.reduce(ncd, dst=0)
                    opcode, check_numel = capi.OP_REDUCE, (total if rank == 0 else 0)
                elif opname == "gather":
                    dst = view(recvbuf, plain_recv, tdt, total)
                    ours = lambda: w.comm.gather(src[:per], dst, per, dt, 0)
                    ncd = nccl_recv.view(tdt)[:total]
                    outs = [ncd[p * per:(p + 1) * per] for p in range(n)] if rank == 0 else None
                    nccl = lambda: dist.gather(ncs[:per], outs, dst=0)
                    opcode, check_numel = capi.OP_GATHER, (total if rank == 0 else 0)
                elif opname == "scatter":
                    dst = view(recvbuf, plain_recv, tdt, per)
                    ours = lambda: w.comm.scatter(src, dst, per, dt, 0)
                    ncd = nccl_recv.view(tdt)[:per]
                    ins = [ncs[p * per:(p + 1) * per] for p in range(n)] if rank == 0 else None
                    nccl = lambda: dist.scatter(ncd, ins, src=0)
                    opcode, check_numel = capi.OP_SCATTER, per
                elif opname == "alltoallv":
                    counts = uneven_counts(max(per // 2, 1), n)
                    sc, rc = counts[rank], [counts[p][rank] for p in range(n)]
                    sd = [sum(sc[:i]) for i in range(n)]
                    rd = [sum(rc[:i]) for i in range(n)]
                    dst = view(recvbuf, plain_recv, tdt, max(sum(rc), 1))
                    src_v = view(sendbuf, plain_send, tdt, max(sum(sc), total))
                    ours = lambda: w.comm.all_to_allv(src_v, sc, sd, dst, rc, rd, dt)
                    ncd = nccl_recv.view(tdt)[:sum(rc)]
                    ncs_v = nccl_send.view(tdt)[:sum(sc)]
                    ncs_v.copy_(src_v[:sum(sc)])
                    nccl = lambda: dist.all_to_all_single(ncd, ncs_v, rc, sc)
                    opcode, check_numel, moved = capi.OP_ALLTOALLV, sum(rc), sum(sc)
                elif opname == "sendrecv":
                    dst = view(recvbuf, plain_recv, tdt, total)

                    def ours():
                        w.comm.group_start()
                        w.comm.send(src, total, dt, (rank + 1) % n)
                        w.comm.recv(dst, total, dt, (rank - 1) % n)
                        w.comm.group_end()
                    ncd = nccl_recv.view(tdt)[:total]

                    def nccl():
                        ops = [dist.P2POp(dist.isend, ncs, (rank + 1) % n), dist.P2POp(dist.irecv, ncd, (rank - 1) % n)]
                        for wk in dist.batch_isend_irecv(ops):
                            wk.wait()
                    opcode = capi.OP_SEND
                elif opname == "putsignal":
                    if plain:
                        break  # needs a registered window on the receiving side
                    dst = recvbuf.view(tdt, total)
                    desc = capi.WaitSignalDesc(1, (rank - 1) % n)

                    def ours():  # put into the next rank's window, then wait for the previous rank's put
                        capi.check(capi.lib().flagcxPutSignal(capi._ptr(src), capi.C.c_size_t(total), dt, (rank + 1) % n,
                                                              recvbuf.win, capi.C.c_size_t(0), 0, w.comm.h, None), "flagcxPutSignal", w.comm.h)
                        capi.check(capi.lib().flagcxWaitSignal(1, capi.C.byref(desc), w.comm.h, None), "flagcxWaitSignal", w.comm.h)
                    ncd = nccl_recv.view(tdt)[:total]

                    def nccl():  # closest NCCL shape: a ring send/recv
                        ops = [dist.P2POp(dist.isend, ncs, (rank + 1) % n), dist.P2POp(dist.irecv, ncd, (rank - 1) % n)]
                        for wk in dist.batch_isend_irecv(ops):
                            wk.wait()
                    opcode = capi.OP_SEND
                else:
                    raise SystemExit(f"unknown op {opname}")
                factor = factor_of(opname, n)
                # correctness against NCCL on the same inputs
                if ours_prep:
                    ours_prep()
                ours()
                ok = True
                if not args.no_nccl and nccl is not None:
                    if nccl_prep:
                        nccl_prep()
                    nccl()
                    torch.cuda.synchronize()
                    if check_numel:
                        a, b = dst[:check_numel].float(), ncd[:check_numel].float()
                        tol = (2 ** -6 if dtn == "bf16" else 1e-5) * max(1, n // 2)
                        ok = bool(((a - b).abs() <= tol * b.abs().clamp(min=1)).all())
                torch.cuda.synchronize()
                assert w.comm.async_error() == 0, w.comm.last_error()
                t_ours = timer.run(ours, ours_prep)
                t_nccl = float("nan") if (args.no_nccl or nccl is None) else timer.run(nccl, nccl_prep)
                nbytes = moved * es
                st = w.comm.stats(opcode)
                row = {"impl": "ours", "op": opname + ("_fused" if args.fused and opname == "allreduce" else ""),
                       "dtype": dtn, "bytes": nbytes, "n_gpus": n, "mode": args.mode, "ours_us": t_ours, "nccl_us": t_nccl,
                       "ours_busbw": nbytes / t_ours / 1e3 * factor, "nccl_busbw": nbytes / t_nccl / 1e3 * factor,
                       "algo": st.lastAlgo, "nctas": st.lastCtas, "correct": ok, "registered": not plain}
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
    ub = w.comm.user_buffer_stats()
    if rank == 0:
        print(f"# user buffers: exports {ub.exports} hits {ub.hits} refused {ub.refused} stale {ub.stale}", flush=True)
    torch.cuda.synchronize()
    dist.barrier()
    if put_win is not None:
        w.comm.window_deregister(put_win)
    for b in (sendbuf, recvbuf):
        if b is not None:
            b.free()
    if plain:
        tb.unfollow_torch_allocator(w.comm)
    w.comm.destroy()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "ours_pg", "nccl", "reference"])
    ap.add_argument("--ref-dir", default="baseline/_ref")
    ap.add_argument("--ops", default="allreduce,reducescatter,allgather,alltoall")
    ap.add_argument("--dtypes", default="bf16,fp32")
    ap.add_argument("--min-bytes", default="1K")
    ap.add_argument("--max-bytes", default="256M")
    ap.add_argument("--mode", default="bandwidth", choices=["bandwidth", "latency"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--no-nccl", action="store_true")
    ap.add_argument("--plain", "--staged", dest="plain", action="store_true",
                    help="ordinary torch tensors instead of registered windows")
    ap.add_argument("--fused", action="store_true", help="allreduce variant with scale=1/world and bf16->fp32 cast in-kernel")
    ap.add_argument("--tune", action="store_true", help="run the tuner over the sweep range first")
    ap.add_argument("--algo", type=int, default=-1)
    ap.add_argument("--nctas", type=int, default=0)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    if args.ops == "all":
        args.ops = ",".join(ALL_OPS)
    if args.impl == "ours":
        run_capi_arm(args)
    else:
        run_pg_arm(args)


if __name__ == "__main__":
    main()
