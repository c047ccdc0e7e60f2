"""Tensor-parallel MLP of a Llama-3-70B-shaped layer (hidden 8192, FFN 28672, 8192
tokens, bf16): the fused kernels of this repository against NCCL + cuBLAS.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29503 bench/tp_layer.py

  column-parallel  all-gather(X shards) -> X[8192,8192] @ W1_r[FFN/N,8192].T
                   ours: one kernel (flagcxTpAllGatherGemm); baseline: all_gather_into_tensor + matmul
  row-parallel     H_r[8192,FFN/N] @ W2_r[8192,FFN/N].T -> reduce-scatter over rows
                   ours: one kernel (flagcxTpGemmReduceScatter); baseline: matmul + reduce_scatter_tensor
  plain GEMM       the tcgen05 kernel alone against cuBLAS (torch.matmul) on the same shape

Weights N(0, 0.02), activations N(0,1), seed = rank.  CUDA events, L2 flush between
iterations, median, max over ranks.  Roofline of a fused op = max(FLOPs / measured
cuBLAS peak, NVLink bytes per rank and direction / 770 GB/s).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flagcx_b200.parallel.tp import AllGatherGemm, GemmReduceScatter, gemm_bf16  # noqa: E402
from flagcx_b200.utils.dist import init_world, max_over_ranks  # noqa: E402


def timed(fn, iters, warmup, flush, world):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.add_(1)
        if world > 1:
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
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--ffn", type=int, default=28672)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    w = init_world()
    n, rank = w.world, w.rank
    M, Hd, F = args.tokens, args.hidden, args.ffn // n
    peaks = {"bf16_tflops": 1672.3}
    try:
        with open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except OSError:
        pass
    peak = peaks["bf16_tflops"] * 1e12
    flush = torch.zeros(64 << 20, dtype=torch.float32, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(rank)
    res = {"n_gpus": n, "tokens": M, "hidden": Hd, "ffn_per_rank": F, "peak_tflops_used": peaks["bf16_tflops"]}

    # ---- plain GEMM: tcgen05 kernel against cuBLAS ----
    a = torch.randn(M, Hd, generator=g, device="cuda").to(torch.bfloat16)
    w1 = (torch.randn(F, Hd, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    out = torch.empty(M, F, dtype=torch.bfloat16, device="cuda")
    flops = 2.0 * M * F * Hd
    t_ours = timed(lambda: gemm_bf16(a, w1, out), args.iters, args.warmup, flush, n)
    t_cublas = timed(lambda: torch.matmul(a, w1.T, out=out), args.iters, args.warmup, flush, n)
    res["gemm"] = {"shape": [M, F, Hd], "ours_us": t_ours, "cublas_us": t_cublas,
                   "ours_tflops": flops / t_ours / 1e6, "cublas_tflops": flops / t_cublas / 1e6,
                   "frac_of_measured_peak": flops / t_ours / 1e-6 / peak}

    if n > 1:
        rows = M // n
        # ---- column-parallel: all-gather -> GEMM ----
        x_shard = torch.randn(rows, Hd, generator=g, device="cuda").to(torch.bfloat16)
        agg = AllGatherGemm(w.comm, M, F, Hd)
        agg.shard.copy_(x_shard)
        gathered = torch.empty(M, Hd, dtype=torch.bfloat16, device="cuda")
        d_ours = torch.empty(M, F, dtype=torch.bfloat16, device="cuda")
        d_ref = torch.empty(M, F, dtype=torch.bfloat16, device="cuda")

        def base_ag():
            dist.all_gather_into_tensor(gathered, x_shard)
            torch.matmul(gathered, w1.T, out=d_ref)

        agg(w1, d_ours)
        base_ag()
        torch.cuda.synchronize()
        ok1 = bool(((d_ours.float() - d_ref.float()).abs() <= 0.02 * (d_ref.float().abs() + d_ref.float().abs().mean())).all())
        t_f = timed(lambda: agg(w1, d_ours), args.iters, args.warmup, flush, n)
        t_b = timed(base_ag, args.iters, args.warmup, flush, n)
        link_bytes = (n - 1) * rows * Hd * 2  # bytes each rank must receive
        roof = max(flops / peak, link_bytes / 770e9)
        res["ag_gemm"] = {"fused_us": t_f, "nccl_cublas_us": t_b, "speedup": t_b / t_f, "correct": ok1,
                          "roofline_us": roof * 1e6, "frac_of_roofline": roof * 1e6 / t_f}
        agg.close()
        # ---- row-parallel: GEMM -> reduce-scatter ----
        h = torch.randn(M, F, generator=g, device="cuda").to(torch.bfloat16)
        w2 = (torch.randn(Hd, F, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
        grs = GemmReduceScatter(w.comm, M, Hd, F)
        o_ours = torch.empty(rows, Hd, dtype=torch.bfloat16, device="cuda")
        o_ref = torch.empty(rows, Hd, dtype=torch.bfloat16, device="cuda")
        full = torch.empty(M, Hd, dtype=torch.bfloat16, device="cuda")

        def base_rs():
            torch.matmul(h, w2.T, out=full)
            dist.reduce_scatter_tensor(o_ref, full)

        grs(h, w2, o_ours)
        base_rs()
        torch.cuda.synchronize()
        ok2 = bool(((o_ours.float() - o_ref.float()).abs() <= 0.03 * (o_ref.float().abs() + o_ref.float().abs().mean())).all())
        flops2 = 2.0 * M * Hd * F
        t_f = timed(lambda: grs(h, w2, o_ours), args.iters, args.warmup, flush, n)
        t_b = timed(base_rs, args.iters, args.warmup, flush, n)
        link_bytes = (n - 1) * rows * Hd * 2
        roof = max(flops2 / peak, link_bytes / 770e9)
        res["gemm_rs"] = {"fused_us": t_f, "nccl_cublas_us": t_b, "speedup": t_b / t_f, "correct": ok2,
                          "roofline_us": roof * 1e6, "frac_of_roofline": roof * 1e6 / t_f}
        grs.close()
        assert w.comm.async_error() == 0, w.comm.last_error()
    if rank == 0:
        print(json.dumps(res), flush=True)
        if args.out:
            os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
            with open(args.out, "w") as f:
                f.write(json.dumps(res) + "\n")
    torch.cuda.synchronize()
    if n > 1:
        dist.barrier()
    w.comm.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
