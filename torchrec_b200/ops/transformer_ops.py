"""Fused elementwise / normalisation pieces of a transformer block over packed tokens ``[T, D]`` (CUDA: ``transformer_kernels.cu``;
elsewhere plain torch, which is also the oracle of the kernel tests).

``residual_layer_norm(a, r, weight, bias, p)`` returns ``(s, y)`` with ``s = r + dropout(a)`` (the residual stream, ``a`` may be
``None``) and ``y = layer_norm(s)``: one pass instead of dropout + add + layer norm, in bf16 with fp32 statistics.
``gelu_dropout(z, p)`` is ``dropout(gelu(z))``.  Dropout masks are recomputed from a per-call seed in the backward instead of being
stored.
"""
from __future__ import annotations

import itertools
from typing import Optional, Tuple

import torch

from torchrec_b200.ops import _ext

_seed_counter = itertools.count(0x5EED)


def _next_seed() -> int:
    """A fresh dropout seed per call, derived from torch's generator so that ``torch.manual_seed`` makes runs repeatable."""
    base = int(torch.initial_seed()) & 0x7FFFFFFF
    return (base * 1_000_003 + next(_seed_counter)) & 0x7FFFFFFFFFFFFFFF


def _kernel_ok(r: torch.Tensor) -> bool:
    return (r.is_cuda and _ext.has_cuda_ext() and r.dtype == torch.bfloat16 and r.dim() == 2 and r.is_contiguous()
            and r.shape[1] % 256 == 0 and r.shape[1] <= 1024)


class _ResidualLayerNorm(torch.autograd.Function):
    """(a, r) -> (s, y): both outputs carry gradient (s feeds the next residual connection, y the next sub-block)."""

    @staticmethod
    def forward(ctx, a, r, weight, bias, p: float, eps: float):
        seed = _next_seed()
        s, y, mean, rstd = torch.ops.trb200.ln_residual_fwd(a, r, weight.float(), bias.float(), p, seed, eps)
        ctx.save_for_backward(s, weight, mean, rstd)
        ctx.cfg = (p, seed)
        return s, y

    @staticmethod
    def backward(ctx, ds_extra, dy):
        s, weight, mean, rstd = ctx.saved_tensors
        p, seed = ctx.cfg
        dy = torch.zeros_like(s) if dy is None else dy.contiguous().to(torch.bfloat16)
        extra = None if ds_extra is None else ds_extra.contiguous().to(torch.bfloat16)
        ds, da, dgamma, dbeta = torch.ops.trb200.ln_residual_bwd(extra, dy, s, weight.float(), mean, rstd, p, seed, True)
        return da, ds, dgamma.to(weight.dtype), dbeta.to(weight.dtype), None, None


class _LayerNorm(torch.autograd.Function):
    """r -> layer_norm(r): the same kernels without the dropout-add half."""

    @staticmethod
    def forward(ctx, r, weight, bias, eps: float):
        _, y, mean, rstd = torch.ops.trb200.ln_residual_fwd(None, r, weight.float(), bias.float(), 0.0, 0, eps)
        ctx.save_for_backward(r, weight, mean, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        r, weight, mean, rstd = ctx.saved_tensors
        ds, _, dgamma, dbeta = torch.ops.trb200.ln_residual_bwd(None, dy.contiguous().to(torch.bfloat16), r, weight.float(), mean, rstd, 0.0, 0, False)
        return ds, dgamma.to(weight.dtype), dbeta.to(weight.dtype), None


def residual_layer_norm(a: Optional[torch.Tensor], r: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, p: float = 0.0,
                        training: bool = True, eps: float = 1e-5) -> Tuple[torch.Tensor, torch.Tensor]:
    """``s = r + dropout(a, p)`` (``a`` may be ``None``), ``y = layer_norm(s) * weight + bias``; returns ``(s, y)``."""
    p = float(p) if training else 0.0
    if _kernel_ok(r) and (a is None or (a.shape == r.shape and a.dtype == r.dtype)):
        if a is None:
            return r, _LayerNorm.apply(r, weight, bias, eps)
        return _ResidualLayerNorm.apply(a.contiguous(), r, weight, bias, p, eps)
    s = r if a is None else r + torch.nn.functional.dropout(a, p, training=p > 0)
    y = torch.nn.functional.layer_norm(s.float(), (s.shape[-1],), weight.float(), bias.float(), eps).to(s.dtype)
    return s, y


class _GeluDropout(torch.autograd.Function):
    @staticmethod
    def forward(ctx, z, p: float):
        seed = _next_seed()
        ctx.save_for_backward(z)
        ctx.cfg = (p, seed)
        return torch.ops.trb200.gelu_dropout_fwd(z, p, seed)

    @staticmethod
    def backward(ctx, dh):
        (z,) = ctx.saved_tensors
        p, seed = ctx.cfg
        return torch.ops.trb200.gelu_dropout_bwd(dh.contiguous().to(torch.bfloat16), z, p, seed), None


def gelu_dropout(z: torch.Tensor, p: float = 0.0, training: bool = True) -> torch.Tensor:
    """``dropout(gelu(z), p)`` (exact erf form)."""
    p = float(p) if training else 0.0
    if z.is_cuda and _ext.has_cuda_ext() and z.dtype == torch.bfloat16 and z.is_contiguous() and z.numel() % 8 == 0:
        return _GeluDropout.apply(z, p)
    return torch.nn.functional.dropout(torch.nn.functional.gelu(z), p, training=p > 0)
