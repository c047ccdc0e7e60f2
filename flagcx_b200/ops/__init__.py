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


class _LinearInto(torch.autograd.Function):
    """y = x @ w.T whose weight gradient is written by the GEMM itself into a buffer the
    caller owns (a slice of a flat gradient buffer), instead of into a fresh tensor that
    would then be copied there.  `sink` is (destination [out, in], callback run once the
    GEMM is queued); the weight's .grad stays None."""

    @staticmethod
    def forward(ctx, x, w, sink):
        ctx.save_for_backward(x, w)
        ctx.sink = sink
        return torch.nn.functional.linear(x, w)

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        dst, done = ctx.sink
        dx = g.matmul(w) if ctx.needs_input_grad[0] else None
        torch.mm(g.reshape(-1, g.shape[-1]).t(), x.reshape(-1, x.shape[-1]), out=dst)
        done()
        return dx, None, None


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """F.linear; if the weight carries a `_grad_sink` its gradient goes straight there."""
    sink = getattr(w, "_grad_sink", None)
    if sink is None:
        return torch.nn.functional.linear(x, w)
    return _LinearInto.apply(x, w, sink)


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
