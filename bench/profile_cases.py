"""Small single-GPU cases of the hot kernels, sized for profiler captures (a few launches,
a few hundred MB on the device at most, inputs larger than the 126 MB L2 where DRAM
figures matter).  Each case also prints its CUDA-event time.

    python bench/profile_cases.py --case gemm            # tcgen05 GEMM 8192 x 3584 x 8192
    python bench/profile_cases.py --case gemm_large      # 8192 x 14336 x 8192 (B larger than L2; 0.6 GB on the device)
    python bench/profile_cases.py --case allreduce       # 8 emulated ranks, two-shot, 32 MiB bf16 each
    python bench/profile_cases.py --case reducescatter   # 8 emulated ranks, 8 x 8 MiB bf16 each
    python bench/profile_cases.py --case allgather       # 8 emulated ranks, push
    python bench/profile_cases.py --case alltoall        # 8 emulated ranks, 8 x 4 MiB blocks each (copyKernelEmu)
    python bench/profile_cases.py --case sendrecv        # 8 emulated ranks, ring of 32 MiB messages (p2pKernelEmu)
    python bench/profile_cases.py --case ll              # 8 emulated ranks, 16 KiB all-reduce, barrier-free (llKernelEmu)
    python bench/profile_cases.py --case ring            # 8 emulated ranks, ring all-reduce of 32 MiB
    python bench/profile_cases.py --case allreduce_cast  # 8 emulated ranks, bf16 in / fp32 out two-shot, 32 MiB
    python bench/profile_cases.py --case putsignal       # 2 emulated ranks, flagcxPutSignal of 64 MiB
    python bench/profile_cases.py --case moe             # 8 emulated ranks, 512 tokens x 7168, top-8 of 256
    python bench/profile_cases.py --case model_kernels   # RMSNorm / SwiGLU / cross-entropy / AdamW / RoPE

The multi-rank cases run as an emulated world: all ranks in one cooperative launch
on one GPU, so "peer" traffic is local HBM traffic there -- they show instruction mix,
occupancy and memory efficiency of the kernels, not NVLink throughput.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flagcx_b200 import capi  # noqa: E402


def timed(fn, reps=3):
    fn()
    torch.cuda.synchronize()
    best = 1e9
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e3)
    return best


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    if args.case in ("gemm", "gemm_large"):
        from flagcx_b200.parallel.tp import gemm_bf16
        M, N, K = (8192, 3584, 8192) if args.case == "gemm" else (8192, 14336, 8192)
        a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        b = (torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16)
        out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        us = timed(lambda: gemm_bf16(a, b, out))
        print(f"gemm {M}x{N}x{K}: {us:.1f} us, {2.0 * M * N * K / us / 1e6:.1f} TFLOP/s")
    elif args.case in ("allreduce", "reducescatter", "allgather"):
        n = 8
        comms = capi.Comm.emu_world(n, 0)
        count = (32 << 20) // 2 if args.case == "allreduce" else (8 << 20) // 2
        total = count if args.case == "allreduce" else count * n
        xs = [torch.randn(total if args.case != "allgather" else count, device="cuda").to(torch.bfloat16) for _ in range(n)]
        outs = [torch.empty(total if args.case != "reducescatter" else count, dtype=torch.bfloat16, device="cuda")
                for _ in range(n)]

        def run():
            for r in range(n):
                if args.case == "allreduce":
                    comms[r].all_reduce_fused(xs[r], outs[r], count, capi.BFLOAT16, capi.SUM, algo=capi.ALGO_TWOSHOT)
                elif args.case == "reducescatter":
                    comms[r].reduce_scatter(xs[r], outs[r], count, capi.BFLOAT16, capi.SUM)
                else:
                    comms[r].all_gather(xs[r], outs[r], count, capi.BFLOAT16, algo=capi.ALGO_PUSH)

        us = timed(run)
        moved = total * 2 * n
        print(f"{args.case} emulated x{n}: {us:.1f} us for {moved >> 20} MiB of payload in the world")
        assert comms[0].async_error() == 0
        capi.Comm.emu_world_destroy(comms)
    elif args.case in ("alltoall", "sendrecv", "ll", "ring", "allreduce_cast"):
        n = 8
        comms = capi.Comm.emu_world(n, 0)
        if args.case == "alltoall":
            per = (4 << 20) // 2
            xs = [torch.randn(per * n, device="cuda").to(torch.bfloat16) for _ in range(n)]
            outs = [torch.empty(per * n, dtype=torch.bfloat16, device="cuda") for _ in range(n)]
            run = lambda: [comms[r].all_to_all(xs[r], outs[r], per, capi.BFLOAT16) for r in range(n)]
            moved = per * n * 2 * n
        elif args.case == "sendrecv":
            cnt = (32 << 20) // 2
            xs = [torch.randn(cnt, device="cuda").to(torch.bfloat16) for _ in range(n)]
            outs = [torch.empty(cnt, dtype=torch.bfloat16, device="cuda") for _ in range(n)]

            def run():
                for r in range(n):
                    comms[r].group_start()
                    comms[r].send(xs[r], cnt, capi.BFLOAT16, (r + 1) % n)
                    comms[r].recv(outs[r], cnt, capi.BFLOAT16, (r - 1) % n)
                    comms[r].group_end()
            moved = cnt * 2 * n
        else:
            cnt = (16 << 10) // 2 if args.case == "ll" else (32 << 20) // 2
            xs = [torch.randn(cnt, device="cuda").to(torch.bfloat16) for _ in range(n)]
            cast = args.case == "allreduce_cast"
            outs = [torch.empty(cnt, dtype=torch.float32 if cast else torch.bfloat16, device="cuda") for _ in range(n)]
            algo = {"ll": capi.ALGO_LL, "ring": capi.ALGO_RING, "allreduce_cast": capi.ALGO_TWOSHOT}[args.case]
            run = lambda: [comms[r].all_reduce_fused(xs[r], outs[r], cnt, capi.BFLOAT16, capi.SUM, algo=algo,
                                                     scale=1.0 / n if cast else 1.0,
                                                     out_dtype=capi.FLOAT if cast else capi.NUM_TYPES) for r in range(n)]
            moved = cnt * 2 * n
        us = timed(run)
        print(f"{args.case} emulated x{n}: {us:.1f} us for {moved / (1 << 20):.2f} MiB of payload in the world")
        assert comms[0].async_error() == 0, comms[0].last_error()
        capi.Comm.emu_world_destroy(comms)
    elif args.case == "putsignal":
        n, cnt = 2, (64 << 20) // 2
        comms = capi.Comm.emu_world(n, 0)
        bufs = [torch.zeros(cnt, dtype=torch.bfloat16, device="cuda") for _ in range(n)]
        wins = [comms[r].window_register(bufs[r], cnt * 2) for r in range(n)]
        src = torch.randn(cnt, device="cuda").to(torch.bfloat16)

        def run():  # rank 0 puts into rank 1's window and raises its signal
            capi.check(capi.lib().flagcxPutSignal(capi._ptr(src), capi.C.c_size_t(cnt), capi.BFLOAT16, 1, wins[0],
                                                  capi.C.c_size_t(0), 0, comms[0].h, None), "flagcxPutSignal", comms[0].h)
        us = timed(run)
        print(f"putsignal 64 MiB: {us:.1f} us, {cnt * 2 * 2 / us / 1e3:.0f} GB/s (read + write, one GPU)")
        capi.Comm.emu_world_destroy(comms)
    elif args.case == "moe":
        from flagcx_b200.parallel.moe import MoeDispatcher, route
        n, T, H, E, K = 8, 512, 7168, 256, 8
        comms = capi.Comm.emu_world(n, 0)
        moes = [MoeDispatcher(comms[r], T, H, K, E, T * K * 2) for r in range(n)]
        xs = [torch.randn(T, H, device="cuda").to(torch.bfloat16) for _ in range(n)]
        rt = [route(torch.randn(T, E, device="cuda"), K) for _ in range(n)]
        outs = [torch.empty(T, H, dtype=torch.bfloat16, device="cuda") for _ in range(n)]

        def disp():
            for r in range(n):
                moes[r].dispatch(xs[r], rt[r][0])

        def comb():
            for r in range(n):
                moes[r].combine(rt[r][1], outs[r])

        print(f"moe dispatch emulated x{n}: {timed(disp):.1f} us")
        for r in range(n):
            moes[r].expert_out.copy_(moes[r].recv_rows)
        print(f"moe combine  emulated x{n}: {timed(comb):.1f} us")
        assert comms[0].async_error() == 0
        for m in moes:
            m.close()
        capi.Comm.emu_world_destroy(comms)
    elif args.case == "model_kernels":
        from flagcx_b200 import ops
        T, H, F, V = 4096, 4096, 14336, 128256
        x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
        w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
        us = timed(lambda: ops.ext().rmsnorm_fwd(x, w, 1e-5))
        print(f"rmsnorm_fwd {T}x{H}: {us:.1f} us, {2 * T * H * 2 / us / 1e3:.0f} GB/s")
        _, rstd = ops.ext().rmsnorm_fwd(x, w, 1e-5)
        us = timed(lambda: ops.ext().rmsnorm_bwd(x, x, w, rstd))
        print(f"rmsnorm_bwd {T}x{H}: {us:.1f} us, {3 * T * H * 2 / us / 1e3:.0f} GB/s")
        ab = torch.randn(T, 2 * F, device="cuda").to(torch.bfloat16)
        us = timed(lambda: ops.ext().swiglu_fwd(ab))
        print(f"swiglu_fwd {T}x{F}: {us:.1f} us, {3 * T * F * 2 / us / 1e3:.0f} GB/s")
        logits = torch.randn(T, V, device="cuda").to(torch.bfloat16)
        tgt = torch.randint(0, V, (T,), device="cuda")
        us = timed(lambda: ops.ext().cross_entropy_fwd_bwd_(logits, tgt, 1.0 / T), reps=2)
        print(f"cross_entropy {T}x{V}: {us:.1f} us, {2 * T * V * 2 / us / 1e3:.0f} GB/s (algorithmic: one read, one write)")
        n = 218_112_000  # one Llama-3-8B layer
        p = torch.randn(n, device="cuda").to(torch.bfloat16)
        g = torch.randn(n, device="cuda").to(torch.bfloat16)
        m = torch.zeros_like(p)
        v = torch.zeros_like(p)
        us = timed(lambda: ops.ext().adamw_flat_(p, g, m, v, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1))
        print(f"adamw {n} params: {us:.1f} us, {7 * n * 2 / us / 1e3:.0f} GB/s (4 reads + 3 writes of bf16)")
        q = torch.randn(T, 32, 128, device="cuda").to(torch.bfloat16)
        us = timed(lambda: ops.ext().rope_inplace(q, None, 500000.0, False))
        print(f"rope {T}x32x128 in place: {us:.1f} us, {2 * q.numel() * 2 / us / 1e3:.0f} GB/s")
    else:
        raise SystemExit(f"unknown case {args.case}")


if __name__ == "__main__":
    main()
