"""Reference arm of bench.py: the UNMODIFIED FlagCX torch plugin (installed from the
reference source tree into baseline/_ref) as the torch.distributed backend of a
plain-PyTorch Llama-3-8B-shaped model under torch FSDP (fully_shard), AdamW.

Nothing of this repository's engine, kernels or model code is on this path: the
model below is ordinary torch.nn code, the collectives go through the reference's
ProcessGroup ("flagcx" as registered by the reference package) and from there to
its NCCL adaptor.  Same metric, same shapes, same timing protocol as the main arm.
If the reference package cannot be imported or initialised on this machine the
function reports why and the bench prints {"impl": "reference", "unavailable": ...}.

The same function also serves two comparison arms that isolate what the communication
library alone contributes, since model, FSDP wrapper and optimizer are byte for byte
the ones of the reference arm and only the imported backend differs:
``ours_pg`` (this repository's "flagcx" ProcessGroup) and ``nccl`` (torch's NCCL).
"""
from __future__ import annotations

import os
import sys
import time

REF_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")


def _unavailable(why: str) -> dict:
    return {"impl": "reference", "unavailable": why.replace("\n", " ")[:400]}


def run_reference(args) -> dict:
    return run_torch_fsdp(args, "reference")


def run_torch_fsdp(args, impl: str) -> dict:
    """impl: "reference" (baseline/_ref), "ours_pg" (this repository's backend) or "nccl"."""
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if impl == "reference" and not os.path.isdir(os.path.join(REF_DIR, "flagcx")):
        return _unavailable("baseline/_ref is empty: the reference package was not installed") if rank == 0 else {}
    try:
        import torch
        import torch.distributed as dist
        import torch.nn as nn
        import torch.nn.functional as F
        if impl == "reference":
            sys.path.insert(0, REF_DIR)
            os.environ.setdefault("TORCH_DEVICE_BACKEND_AUTOLOAD", "0")
            import flagcx  # noqa: F401  the reference's package; registers backend "flagcx"
            if hasattr(flagcx, "init"):
                flagcx.init()
        elif impl == "ours_pg":
            sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
            import flagcx_b200.torch_backend  # noqa: F401  registers this repository's backend "flagcx"
    except Exception as e:  # noqa: BLE001
        return _unavailable(f"importing the {impl} torch plugin failed: {e!r}") if rank == 0 else {}
    backend_name = "nccl" if impl == "nccl" else "flagcx"

    from torch.distributed.fsdp import fully_shard

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29534")
    try:
        dist.init_process_group(backend_name, rank=rank, world_size=world)
        probe = torch.ones(8, device=dev)
        dist.all_reduce(probe)
        torch.cuda.synchronize()
    except Exception as e:  # noqa: BLE001
        return _unavailable(f"the reference backend failed to initialise: {e!r}") if rank == 0 else {}

    H, NH, NKV, FFN, V, L = (4096, 32, 8, 14336, 128256, 32) if args.model == "llama3_8b" else (256, 4, 2, 512, 1024, 2)
    HD = H // NH
    seq = args.seq_len

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.attn_norm = nn.RMSNorm(H, eps=1e-5)
            self.wqkv = nn.Linear(H, H + 2 * NKV * HD, bias=False)
            self.wo = nn.Linear(H, H, bias=False)
            self.ffn_norm = nn.RMSNorm(H, eps=1e-5)
            self.w13 = nn.Linear(H, 2 * FFN, bias=False)
            self.w2 = nn.Linear(FFN, H, bias=False)

        def forward(self, x, cos, sin):
            B, T, _ = x.shape
            q, k, v = self.wqkv(self.attn_norm(x)).split([NH * HD, NKV * HD, NKV * HD], -1)
            q = q.view(B, T, NH, HD).transpose(1, 2)
            k = k.view(B, T, NKV, HD).transpose(1, 2)
            v = v.view(B, T, NKV, HD).transpose(1, 2)

            def rot(t):
                t1, t2 = t[..., : HD // 2], t[..., HD // 2:]
                return torch.cat([t1 * cos - t2 * sin, t2 * cos + t1 * sin], -1)

            a = F.scaled_dot_product_attention(rot(q), rot(k), v, is_causal=True, enable_gqa=True)
            x = x + self.wo(a.transpose(1, 2).reshape(B, T, H))
            a, b = self.w13(self.ffn_norm(x)).chunk(2, -1)
            return x + self.w2(F.silu(a) * b)

    class Model(nn.Module):
        def __init__(self):
            super().__init__()
            self.embed = nn.Embedding(V, H)
            self.layers = nn.ModuleList([Block() for _ in range(L)])
            self.norm = nn.RMSNorm(H, eps=1e-5)
            self.out = nn.Linear(H, V, bias=False)

        def forward(self, tokens, targets):
            T = tokens.shape[1]
            inv = 500000.0 ** (-torch.arange(0, HD // 2, device=tokens.device, dtype=torch.float32) * 2 / HD)
            ang = torch.arange(T, device=tokens.device, dtype=torch.float32)[:, None] * inv[None]
            cos, sin = ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)
            x = self.embed(tokens)
            for layer in self.layers:
                x = layer(x, cos, sin)
            logits = self.out(self.norm(x))
            return F.cross_entropy(logits.float().view(-1, V), targets.view(-1))

    try:
        torch.manual_seed(1234)
        with torch.device(dev):
            model = Model().to(torch.bfloat16)
        for p in model.parameters():
            if p.dim() > 1:
                nn.init.normal_(p, 0.0, 0.02)
        for layer in model.layers:
            fully_shard(layer)
        fully_shard(model)
        opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)

        total = args.steps + args.warmup
        g = torch.Generator().manual_seed(1000 + rank)
        host = [torch.randint(0, V, (1, seq + 1), generator=g, dtype=torch.long).pin_memory() for _ in range(total)]
        devb = [b.to(dev) for b in host]

        def step(b):
            loss = model(b[:, :-1], b[:, 1:])
            loss.backward()
            opt.step()
            opt.zero_grad(set_to_none=True)
            return loss

        def sync_all():
            torch.cuda.synchronize(dev)
            dist.barrier()
            torch.cuda.synchronize(dev)

        def max_ranks(x):
            t = torch.tensor([x], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())

        for i in range(args.warmup):
            step(host[i].to(dev, non_blocking=True)).item()
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            loss = step(devb[args.warmup + i])
        e1.record()
        sync_all()
        dev_ms = max_ranks(e0.elapsed_time(e1))
        t0 = time.perf_counter()
        for i in range(args.steps):
            last = step(host[args.warmup + i].to(dev, non_blocking=True)).item()
        torch.cuda.synchronize(dev)
        e2e_ms = max_ranks((time.perf_counter() - t0) * 1e3)
    except Exception as e:  # noqa: BLE001
        return _unavailable(f"training through the reference backend failed: {e!r}") if rank == 0 else {}

    if impl == "ours_pg" and rank == 0:
        # how many allocations the backend mapped into the peers, and how often a collective
        # found its buffer already mapped (stderr: the JSON line stays alone on stdout)
        import flagcx_b200.torch_backend as tb
        st = tb.comm_of(dist.group.WORLD, dev).user_buffer_stats()
        print(f"[ours_pg] user buffers: exports {st.exports} hits {st.hits} refused {st.refused} stale {st.stale}",
              file=sys.stderr, flush=True)
    tokens = world * seq * args.steps
    out = {
        "metric": "training tokens/s (Llama-3-8B shape, FSDP full-shard, bf16)",
        "value": tokens / (dev_ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform-random token ids, random-init weights",
        "impl": impl,
        "config": {"model": args.model, "global_batch": world, "seq_len": seq, "parallelism": f"fsdp{world}",
                   "optimizer": "AdamW, fused kernel, bf16 states",
                   "l2": "no flush needed: each step streams 16 GB of parameters plus activations, far above the 126 MB L2"},
        "backend": {"reference": "reference FlagCX torch plugin (NCCL adaptor) + torch fully_shard + fused AdamW",
                    "ours_pg": "this repository's flagcx ProcessGroup + torch fully_shard + fused AdamW",
                    "nccl": "torch NCCL ProcessGroup + torch fully_shard + fused AdamW"}[impl],
        "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                "h2d_bytes_per_step": (seq + 1) * 8, "d2h_bytes_per_step": 4},
        "loss_last": float(last),
    }
    dist.barrier()
    dist.destroy_process_group()
    return out if rank == 0 else {}
