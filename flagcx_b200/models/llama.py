"""Llama-3-shaped decoder written as pure functions over explicit parameter lists.

The model is cut into *units* (embedding, each decoder layer, output head).  A unit
declares the shapes of its parameters and a function ``fn(params, x, ...)``; the
sharding engine (``flagcx_b200.parallel.fsdp``) owns the storage, hands the unit
views of an all-gathered flat buffer, and collects the gradients.  GEMMs and
attention go to the library kernels behind torch (cuBLAS, SDPA); normalisation,
rotary embedding, SwiGLU and the loss are this package's fused kernels.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Callable, List, Sequence, Tuple

import torch
import torch.nn.functional as F

from flagcx_b200 import ops


@dataclass
class LlamaConfig:
    n_layers: int = 32
    hidden: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 8
    ffn: int = 14336
    vocab: int = 128256
    rope_theta: float = 500000.0
    eps: float = 1e-5
    init_std: float = 0.02

    @property
    def head_dim(self) -> int:
        return self.hidden // self.n_heads

    def num_params(self) -> int:
        return sum(sum(_numel(s) for _, s in u.shapes) for u in build_units(self))

    @staticmethod
    def llama3_8b() -> "LlamaConfig":
        return LlamaConfig()

    @staticmethod
    def tiny(vocab: int = 1024) -> "LlamaConfig":
        return LlamaConfig(n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, ffn=512, vocab=vocab)


def _numel(shape: Sequence[int]) -> int:
    n = 1
    for s in shape:
        n *= s
    return n


@dataclass
class Unit:
    name: str
    shapes: List[Tuple[str, Tuple[int, ...]]]
    fn: Callable  # fn(params: list[Tensor], x, *extra) -> Tensor
    init: Callable[[str, torch.Tensor], None]


def _embed_fn(params, tokens):
    (w,) = params
    return F.embedding(tokens, w)


def _make_layer_fn(cfg: LlamaConfig):
    nh, nkv, hd = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim

    def layer(params, x):
        attn_norm, wqkv, wo, ffn_norm, w13, w2 = params
        T = x.shape[0]
        h, skip = ops.rmsnorm_branch(x, attn_norm, cfg.eps)
        qkv = ops.rope_fused_qkv(ops.linear(h, wqkv), nh, nkv, hd, cfg.rope_theta)
        q, k, v = qkv.split([nh * hd, nkv * hd, nkv * hd], dim=-1)  # views: attention reads them strided
        q, k, v = q.view(T, nh, hd), k.view(T, nkv, hd), v.view(T, nkv, hd)
        a = F.scaled_dot_product_attention(q.transpose(0, 1).unsqueeze(0), k.transpose(0, 1).unsqueeze(0),
                                           v.transpose(0, 1).unsqueeze(0), is_causal=True, enable_gqa=True)
        a = a.squeeze(0).transpose(0, 1).reshape(T, nh * hd)
        x = ops.linear(a, wo, residual=skip)
        h, skip = ops.rmsnorm_branch(x, ffn_norm, cfg.eps)
        x = ops.linear(ops.swiglu(ops.linear(h, w13)), w2, residual=skip)
        return x

    def layer_unfused(params, x):
        """The same block from one kernel per operation (separate q / k rotations on copies,
        residual adds as their own kernels): the comparison arm of FLAGCX_MODEL_FUSED=0."""
        attn_norm, wqkv, wo, ffn_norm, w13, w2 = params
        T = x.shape[0]
        h = ops.rmsnorm(x, attn_norm, cfg.eps)
        qkv = ops.linear(h, wqkv)
        q, k, v = qkv.split([nh * hd, nkv * hd, nkv * hd], dim=-1)
        q = ops.rope(q.reshape(T, nh, hd), cfg.rope_theta)
        k = ops.rope(k.reshape(T, nkv, hd), cfg.rope_theta)
        v = v.reshape(T, nkv, hd)
        a = F.scaled_dot_product_attention(q.transpose(0, 1).unsqueeze(0), k.transpose(0, 1).unsqueeze(0),
                                           v.transpose(0, 1).unsqueeze(0), is_causal=True, enable_gqa=True)
        a = a.squeeze(0).transpose(0, 1).reshape(T, nh * hd)
        x = x + ops.linear(a, wo)
        h = ops.rmsnorm(x, ffn_norm, cfg.eps)
        x = x + ops.linear(ops.swiglu(ops.linear(h, w13)), w2)
        return x

    if os.environ.get("FLAGCX_MODEL_FUSED", "1") == "0":
        return layer_unfused
    return layer


def _make_head_fn(cfg: LlamaConfig):
    def head(params, x, targets):
        norm, w = params
        h = ops.rmsnorm(x, norm, cfg.eps)
        logits = ops.linear(h, w)
        return ops.cross_entropy_(logits, targets)

    return head


def build_units(cfg: LlamaConfig) -> List[Unit]:
    std = cfg.init_std

    def init(name: str, t: torch.Tensor) -> None:
        if "norm" in name:
            t.fill_(1.0)
        else:
            t.normal_(0.0, std)

    units = [Unit("embed", [("tok_embeddings", (cfg.vocab, cfg.hidden))], _embed_fn, init)]
    layer_fn = _make_layer_fn(cfg)
    kvd = cfg.n_kv_heads * cfg.head_dim
    for i in range(cfg.n_layers):
        units.append(Unit(f"layer{i}", [
            ("attn_norm", (cfg.hidden,)),
            ("wqkv", (cfg.hidden + 2 * kvd, cfg.hidden)),
            ("wo", (cfg.hidden, cfg.hidden)),
            ("ffn_norm", (cfg.hidden,)),
            ("w13", (2 * cfg.ffn, cfg.hidden)),
            ("w2", (cfg.hidden, cfg.ffn)),
        ], layer_fn, init))
    units.append(Unit("head", [("norm", (cfg.hidden,)), ("output", (cfg.vocab, cfg.hidden))], _make_head_fn(cfg), init))
    return units


def reference_forward(cfg: LlamaConfig, flat_params: List[List[torch.Tensor]], tokens: torch.Tensor,
                      targets: torch.Tensor) -> torch.Tensor:
    """The same network in plain PyTorch fp32 ops (no custom kernels): the oracle the
    tests compare the fused kernels and the sharded engine against."""
    def rms(x, w):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + cfg.eps) * w.float())

    def rope(x):
        T, H, D = x.shape
        half = D // 2
        inv = cfg.rope_theta ** (-torch.arange(0, half, device=x.device, dtype=torch.float32) * 2 / D)
        ang = torch.arange(T, device=x.device, dtype=torch.float32)[:, None] * inv[None, :]
        c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
        x1, x2 = x[..., :half].float(), x[..., half:].float()
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)

    nh, nkv, hd = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
    x = F.embedding(tokens, flat_params[0][0].float())
    for params in flat_params[1:-1]:
        attn_norm, wqkv, wo, ffn_norm, w13, w2 = [p.float() for p in params]
        T = x.shape[0]
        h = rms(x, attn_norm)
        q, k, v = (h @ wqkv.T).split([nh * hd, nkv * hd, nkv * hd], -1)
        q, k, v = rope(q.reshape(T, nh, hd)), rope(k.reshape(T, nkv, hd)), v.reshape(T, nkv, hd)
        k = k.repeat_interleave(nh // nkv, 1)
        v = v.repeat_interleave(nh // nkv, 1)
        att = torch.einsum("qhd,khd->hqk", q, k) / hd ** 0.5
        att = att.masked_fill(torch.ones(T, T, device=x.device).triu(1).bool(), float("-inf")).softmax(-1)
        a = torch.einsum("hqk,khd->qhd", att, v).reshape(T, nh * hd)
        x = x + a @ wo.T
        h = rms(x, ffn_norm)
        ab = h @ w13.T
        x = x + (F.silu(ab[:, :cfg.ffn]) * ab[:, cfg.ffn:]) @ w2.T
    norm, w = [p.float() for p in flat_params[-1]]
    logits = rms(x, norm) @ w.T
    return F.cross_entropy(logits, targets)
