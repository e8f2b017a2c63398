"""Fused elementwise / normalisation pieces of a transformer block over packed tokens ``[T, D]`` (CUDA: ``transformer_kernels.cu``;
elsewhere plain torch, which is also the oracle of the kernel tests).

``residual_layer_norm(a, r, weight, bias, p)`` returns ``(s, y)`` with ``s = r + dropout(a)`` (the residual stream, ``a`` may be
``None``) and ``y = layer_norm(s)``: one pass instead of dropout + add + layer norm, in bf16 with fp32 statistics.
``gelu_dropout(z, p)`` is ``dropout(gelu(z))``.  Dropout masks are recomputed from a per-call seed in the backward instead of being
stored.  ``packed_attention(qkv, offsets, heads, max_len, p)`` is self-attention inside every sequence of packed tokens
(``varlen_attention.cu``).  ``sampled_softmax_loss(h, positive, negatives)`` is the cross entropy of a sampled softmax with its
gradient produced in the same pass over the scores (``sampled_softmax_kernels.cu``).
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


# --------------------------------------------------------------------------------------
# attention over packed sequences
# --------------------------------------------------------------------------------------
ATTENTION_HEAD_DIM = 64     # the kernel's head dimension
ATTENTION_MAX_LEN = 768     # longest sequence whose K and V (or Q and dO) fit in one CTA's shared memory
_attn_err: dict = {}


def _attention_error_word(device: torch.device) -> torch.Tensor:
    word = _attn_err.get(device)
    if word is None:
        word = _attn_err[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return word


def attention_error(device: torch.device) -> int:
    """Non-zero after a packed-attention launch met a sequence longer than its ``max_len`` (the tail of that sequence got zeros).
    Reading it synchronises with the device."""
    word = _attn_err.get(torch.device(device))
    return 0 if word is None else int(word.item())


def packed_attention_supported(qkv: torch.Tensor, num_heads: int, max_len: int) -> bool:
    return (qkv.is_cuda and _ext.has_cuda_ext() and qkv.dtype == torch.bfloat16 and qkv.dim() == 2 and qkv.shape[1] == 3 * num_heads * ATTENTION_HEAD_DIM
            and 1 <= max_len <= ATTENTION_MAX_LEN)


class _PackedAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, offsets, num_heads: int, max_len: int, p: float):
        seed = _next_seed() if p > 0 else 0
        err = _attention_error_word(qkv.device)
        out, lse = torch.ops.trb200.varlen_attn_fwd(qkv, offsets, num_heads, max_len, p, seed, err)
        ctx.save_for_backward(qkv, out, lse, offsets)
        ctx.cfg = (num_heads, max_len, p, seed)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse, offsets = ctx.saved_tensors
        num_heads, max_len, p, seed = ctx.cfg
        dqkv = torch.ops.trb200.varlen_attn_bwd(dout.contiguous().to(torch.bfloat16), qkv, out, lse, offsets, num_heads, max_len, p, seed,
                                                _attention_error_word(qkv.device))
        return dqkv, None, None, None, None


def packed_attention(qkv: torch.Tensor, offsets: torch.Tensor, num_heads: int, max_len: int, p: float = 0.0) -> torch.Tensor:
    """Self-attention inside every sequence of the packed ``qkv [T, 3 * D]`` (``q | k | v`` along the columns, head dimension 64,
    bf16); ``offsets [B + 1]`` bounds the sequences, none longer than ``max_len``.  Returns ``[T, D]``; dropout with probability ``p``
    acts on the attention probabilities.  The caller checks ``packed_attention_supported`` first."""
    return _PackedAttention.apply(qkv.contiguous(), offsets.to(torch.int64).contiguous(), int(num_heads), int(max_len), float(p))


# --------------------------------------------------------------------------------------
# sampled softmax
# --------------------------------------------------------------------------------------
class _SampledSoftmaxLoss(torch.autograd.Function):
    """mean_p CE([h_p . pos_p, h_p . neg_0, ..., h_p . neg_{N-1}], class 0).  The scores ``[P, N]`` exist once, in bf16; the kernel
    that reads them for the loss overwrites them with their gradient, which the backward feeds to two GEMMs."""

    @staticmethod
    def forward(ctx, h, positive, negatives):
        from torchrec_b200.ops import dense_ops

        P, D = h.shape
        rows = (P + 7) // 8 * 8  # the weight-gradient GEMM wants a row count that is a multiple of 8: zero rows at the end
        h16 = h.new_zeros(rows, D, dtype=torch.bfloat16)
        h16[:P] = h
        n16 = negatives.to(torch.bfloat16).contiguous()
        scores = dense_ops.gemm_nt(h16, n16)  # [rows, N] bf16
        pos = (h16[:P].float() * positive.float()).sum(-1)
        loss_rows, dpos = torch.ops.trb200.sampled_ce_fwd_bwd(pos, scores, 1.0 / max(P, 1))
        if rows != P:
            scores[P:].zero_()
        ctx.save_for_backward(h16, positive, n16, scores, dpos)
        ctx.P = P
        ctx.dtypes = (h.dtype, positive.dtype, negatives.dtype)
        return loss_rows.sum() / max(P, 1)

    @staticmethod
    def backward(ctx, g):
        from torchrec_b200.ops import dense_ops

        h16, positive, n16, dscores, dpos = ctx.saved_tensors
        P = ctx.P
        dh = dpos_term = dneg = None
        if ctx.needs_input_grad[0]:
            dh = dense_ops.gemm_nt(dscores, n16.t().contiguous())[:P].float() + dpos.unsqueeze(1) * positive.float()
            dh = (dh * g).to(ctx.dtypes[0])
        if ctx.needs_input_grad[1]:
            dpos_term = (dpos.unsqueeze(1) * h16[:P].float() * g).to(ctx.dtypes[1])
        if ctx.needs_input_grad[2]:
            dneg = (dense_ops.gemm_tn(dscores, h16) * g).to(ctx.dtypes[2])
        return dh, dpos_term, dneg


def sampled_softmax_loss(h: torch.Tensor, positive: torch.Tensor, negatives: torch.Tensor) -> torch.Tensor:
    """Mean cross entropy of a sampled softmax: row ``p`` scores its own positive ``positive[p]`` (class 0) and the shared
    ``negatives [N, D]`` against ``h[p]``.  Equal to ``cross_entropy(cat([sum(h * positive, -1, keepdim), h @ negatives.T], 1), 0)``."""
    if (h.is_cuda and _ext.has_cuda_ext() and h.dim() == 2 and h.dtype in (torch.bfloat16, torch.float32) and negatives.shape[0] % 8 == 0
            and negatives.shape[0] >= 8 and h.shape[1] % 8 == 0 and h.shape[0] > 0):
        return _SampledSoftmaxLoss.apply(h, positive, negatives)
    scores = torch.cat([(h * positive.to(h.dtype)).sum(-1, keepdim=True), h @ negatives.to(h.dtype).t()], dim=1).float()
    return torch.nn.functional.cross_entropy(scores, torch.zeros(scores.shape[0], dtype=torch.long, device=scores.device))
