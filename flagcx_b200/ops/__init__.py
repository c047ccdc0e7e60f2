"""Fused CUDA ops with autograd wrappers.

Every function here runs a hand-written sm_100a kernel from ``csrc/`` and raises
if the extension is missing -- there is no eager fallback, so a run that is
supposed to use these kernels cannot silently use something else.
"""
from __future__ import annotations

import importlib.util
import os

import torch

from . import build as _build

_ext = None
launch_count = 0  # kernels launched through this module (bench.py reports it)
# When the loss is only ever differentiated with gradient 1 (loss.backward()), the
# cross-entropy backward can hand out the stored gradient without another pass.
assume_unit_loss_grad = False


def ext():
    global _ext
    if _ext is None:
        path = _build.built_path()
        if path is None:
            if os.environ.get("FLAGCX_TORCH_NO_JIT"):
                raise ImportError("flagcx fused-op extension is not built; run flagcx_b200.build.build()")
            path = _build.build()
        spec = importlib.util.spec_from_file_location(_build.NAME, path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _ext = mod
    return _ext


def _count(n=1):
    global launch_count
    launch_count += n


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        y, rstd = ext().rmsnorm_fwd(x, weight, eps)
        _count()
        ctx.save_for_backward(x, weight, rstd)
        return y

    @staticmethod
    def backward(ctx, g):
        x, weight, rstd = ctx.saved_tensors
        dx, dw = ext().rmsnorm_bwd(g.contiguous(), x, weight, rstd)
        _count()
        return dx, dw, None


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    return _RMSNorm.apply(x.contiguous(), weight, eps)


class _RMSNormBranch(torch.autograd.Function):
    """The pre-norm of a residual block: returns (norm(x), x).  The second output is x itself,
    to be used as the block's skip connection; routing it through this function lets the
    backward add the skip connection's gradient to the norm's input gradient inside the
    RMSNorm backward kernel, where autograd would otherwise launch an add over [T, H]."""

    @staticmethod
    def forward(ctx, x, weight, eps):
        y, rstd = ext().rmsnorm_fwd(x, weight, eps)
        _count()
        ctx.save_for_backward(x, weight, rstd)
        return y, x.view_as(x)

    @staticmethod
    def backward(ctx, g, g_skip):
        x, weight, rstd = ctx.saved_tensors
        if g is None:  # only the skip connection was used
            return g_skip, None, None
        add = g_skip.contiguous() if g_skip is not None else None
        dx, dw = ext().rmsnorm_bwd(g.contiguous(), x, weight, rstd, add)
        _count()
        return dx, dw, None


def rmsnorm_branch(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5):
    """(rmsnorm(x), x): see _RMSNormBranch.  Use the second value for the residual add."""
    return _RMSNormBranch.apply(x.contiguous(), weight, eps)


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, theta):
        ctx.theta = theta
        x = x.contiguous().clone()
        ext().rope_inplace(x, None, theta, False)
        _count()
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        ext().rope_inplace(g, None, ctx.theta, True)
        _count()
        return g, None


def rope(x: torch.Tensor, theta: float = 500000.0) -> torch.Tensor:
    """x: [tokens, heads, head_dim]; token t is at position t (one sequence per call)."""
    return _Rope.apply(x, theta)


class _RopeFusedQkv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, rope_heads, total_heads, head_dim, theta):
        ctx.shape = (rope_heads, total_heads, head_dim, theta)
        _count()
        return ext().rope_fused_qkv(qkv, rope_heads, total_heads, head_dim, theta, False)

    @staticmethod
    def backward(ctx, g):
        rope_heads, total_heads, head_dim, theta = ctx.shape
        _count()
        return ext().rope_fused_qkv(g.contiguous(), rope_heads, total_heads, head_dim, theta, True), None, None, None, None


def rope_fused_qkv(qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, theta: float = 500000.0) -> torch.Tensor:
    """qkv: [tokens, (n_heads + 2 * n_kv_heads) * head_dim] as the fused projection leaves it
    (queries, keys, values side by side).  Rotates the query and key heads (token t at
    position t) and copies the value heads, in one pass; q, k and v are then views of the
    result and no per-tensor copy is needed before attention."""
    return _RopeFusedQkv.apply(qkv.contiguous(), n_heads + n_kv_heads, n_heads + 2 * n_kv_heads, head_dim, theta)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ab):
        ab = ab.contiguous()
        ctx.save_for_backward(ab)
        _count()
        return ext().swiglu_fwd(ab)

    @staticmethod
    def backward(ctx, g):
        (ab,) = ctx.saved_tensors
        _count()
        return ext().swiglu_bwd(g.contiguous(), ab)


def swiglu(ab: torch.Tensor) -> torch.Tensor:
    """ab = [a | b] along the last dimension; returns silu(a) * b."""
    return _SwiGLU.apply(ab)


def _mm_residual(x, w, residual):
    # cuBLAS adds the residual in the GEMM's epilogue (beta = 1): no separate add kernel
    y = torch.addmm(residual.reshape(-1, residual.shape[-1]), x.reshape(-1, x.shape[-1]), w.t())
    return y.view(*x.shape[:-1], w.shape[0])


class _LinearInto(torch.autograd.Function):
    """y = x @ w.T (+ residual) whose weight gradient is written by the GEMM itself into a
    buffer the caller owns (a slice of a flat gradient buffer), instead of into a fresh
    tensor that would then be copied there.  `sink` is (destination [out, in], callback run
    once the GEMM is queued); the weight's .grad stays None."""

    @staticmethod
    def forward(ctx, x, w, sink, residual):
        ctx.save_for_backward(x, w)
        ctx.sink = sink
        if residual is None:
            return torch.nn.functional.linear(x, w)
        return _mm_residual(x, w, residual)

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        dst, done = ctx.sink
        dx = g.matmul(w) if ctx.needs_input_grad[0] else None
        torch.mm(g.reshape(-1, g.shape[-1]).t(), x.reshape(-1, x.shape[-1]), out=dst)
        done()
        return dx, None, None, (g if ctx.needs_input_grad[3] else None)


class _LinearResidual(torch.autograd.Function):
    """y = x @ w.T + residual with the add in the GEMM epilogue; the residual's gradient is
    the incoming gradient itself (no kernel)."""

    @staticmethod
    def forward(ctx, x, w, residual):
        ctx.save_for_backward(x, w)
        return _mm_residual(x, w, residual)

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        dx = g.matmul(w) if ctx.needs_input_grad[0] else None
        dw = g.reshape(-1, g.shape[-1]).t().mm(x.reshape(-1, x.shape[-1])) if ctx.needs_input_grad[1] else None
        return dx, dw, (g if ctx.needs_input_grad[2] else None)


def linear(x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
    """F.linear, optionally with `residual` (same shape as the result) added in the GEMM's
    epilogue; if the weight carries a `_grad_sink` its gradient goes straight there."""
    sink = getattr(w, "_grad_sink", None)
    if sink is None:
        if residual is None:
            return torch.nn.functional.linear(x, w)
        return _LinearResidual.apply(x, w, residual)
    return _LinearInto.apply(x, w, sink, residual)


_unit_grad_checked = False


class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets):
        # the kernel turns `logits` into its own gradient: no second [T, V] tensor
        rows = logits.numel() // logits.size(-1)
        losses = ext().cross_entropy_fwd_bwd_(logits, targets, 1.0 / rows)
        _count()
        # tell autograd the input was overwritten (it then refuses a backward of an
        # upstream op that had saved these logits); a dirty input must also be an output
        ctx.mark_dirty(logits)
        ctx.save_for_backward(logits)
        return losses.mean(), logits

    @staticmethod
    def backward(ctx, g, _unused):
        global _unit_grad_checked
        (dlogits,) = ctx.saved_tensors
        if assume_unit_loss_grad:
            if not _unit_grad_checked:  # one synchronising look, the first time only
                assert float(g) == 1.0, "assume_unit_loss_grad is set but the loss was differentiated with another gradient"
                _unit_grad_checked = True
            return dlogits, None  # loss.backward() with the default gradient of 1
        return dlogits.mul_(g.to(dlogits.dtype)), None


def cross_entropy_(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Mean softmax cross-entropy.  Consumes `logits` (it is overwritten with the gradient)."""
    return _CrossEntropy.apply(logits, targets)[0]


def adamw_flat_(p, g, m, v, lr, beta1, beta2, eps, weight_decay, step) -> None:
    ext().adamw_flat_(p, g, m, v, lr, beta1, beta2, eps, weight_decay, step)
    _count()
