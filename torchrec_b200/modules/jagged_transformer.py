"""A transformer encoder over PACKED tokens: sequences of different lengths lie back to back in one ``[T, D]`` tensor and no
padding position is ever computed.

``jagged_encoder_forward(encoder, x, offsets, max_len)`` runs the layers of an ``nn.TransformerEncoder`` (pre-norm, GELU,
``batch_first``) with the encoder's own parameters, so checkpoints and the padded reference path stay interchangeable:

* projections and feed-forward layers are the tcgen05 GEMMs with bias epilogues (``ops.dense_ops.linear_act``);
* ``dropout + residual add + layer norm`` is one kernel, ``gelu + dropout`` another (``ops.transformer_ops``), with masks recomputed in
  the backward instead of stored;
* attention runs on the packed tokens too: one CTA per (sequence, head) with the sequence's K and V in shared memory
  (``ops.transformer_ops.packed_attention``, head dimension 64, sequences up to 768 tokens).  Other shapes pad q, k, v for one
  library attention call with the padded keys masked (``ATTENTION_MODE = "padded"``; ``"nested"`` selects the library's
  variable-length kernel where the build has one).

With lengths uniform in [20, 200] this is 55 % of the padded token count before any kernel gets faster.  The reference's
BERT4Rec runs padded ``[B, L, D]`` tensors through library modules (``examples/bert4rec/models/bert4rec.py`` of the reference).
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from torchrec_b200.ops import dense_ops
from torchrec_b200.ops.transformer_ops import gelu_dropout, packed_attention, packed_attention_supported, residual_layer_norm


def supports(encoder: nn.TransformerEncoder) -> bool:
    """The packed path covers the configuration the models here build: pre-norm layers with GELU and no custom masks."""
    for layer in encoder.layers:
        if not isinstance(layer, nn.TransformerEncoderLayer) or not layer.norm_first:
            return False
        if getattr(layer, "activation_relu_or_gelu", 0) != 2:
            return False
        if not layer.self_attn._qkv_same_embed_dim or layer.self_attn.in_proj_bias is None:
            return False
    return True


def _attention_per_sequence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, offsets: torch.Tensor, p: float) -> torch.Tensor:
    """Oracle / fallback: one attention call per sequence (``q, k, v [T, H, Dh]``)."""
    out = torch.empty_like(q)
    bounds = offsets.tolist()
    for lo, hi in zip(bounds[:-1], bounds[1:]):
        if hi > lo:
            o = torch.nn.functional.scaled_dot_product_attention(q[lo:hi].transpose(0, 1), k[lo:hi].transpose(0, 1), v[lo:hi].transpose(0, 1), dropout_p=p)
            out[lo:hi] = o.transpose(0, 1)
    return out


def _attention_padded(qkv: torch.Tensor, offsets: torch.Tensor, num_heads: int, max_len: int, p: float) -> torch.Tensor:
    """Attention on a padded view of the packed tokens: only the attention itself sees padding (keys beyond a sequence's length
    are masked out); q, k and v are padded by the jagged-to-padded kernel and the result is packed again."""
    from torchrec_b200.ops import sparse_ops as sops

    T, three_d = qkv.shape
    D = three_d // 3
    B = offsets.numel() - 1
    padded = sops.jagged_to_padded_dense(qkv, offsets, max_len, 0.0)  # [B, L, 3D]
    q, k, v = (t.reshape(B, max_len, num_heads, D // num_heads).transpose(1, 2) for t in padded.split(D, dim=2))
    lengths = (offsets[1:] - offsets[:-1]).clamp(max=max_len)
    key_ok = torch.arange(max_len, device=qkv.device).unsqueeze(0) < lengths.unsqueeze(1)  # [B, L]
    out = torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=key_ok.view(B, 1, 1, max_len), dropout_p=p)
    return sops.padded_dense_to_jagged(out.transpose(1, 2).reshape(B, max_len, D), offsets, T)


ATTENTION_MODE = "kernel"  # "kernel" | "padded" | "nested": how the packed tokens reach an attention kernel on CUDA


def varlen_attention(qkv: torch.Tensor, offsets: torch.Tensor, num_heads: int, max_len: int, p: float = 0.0) -> torch.Tensor:
    """Self-attention inside every sequence of the packed ``qkv [T, 3 * D]``; returns ``[T, D]``.

    ``ATTENTION_MODE = "kernel"`` (default) runs this package's packed-attention kernel where the shape allows (bf16, head
    dimension 64, ``max_len <= 768``; cost ``sum(len^2)``) and the padded form elsewhere.  ``"padded"`` is one library attention
    call over ``[B, H, max_len, Dh]`` with the padded keys masked.  ``"nested"`` hands the packed layout to the library's
    variable-length attention through a jagged nested tensor; where the build has no variable-length kernel for the device that
    silently decomposes into one small attention per sequence.  Everything outside the attention stays packed in every mode."""
    T, three_d = qkv.shape
    D = three_d // 3
    if qkv.is_cuda and ATTENTION_MODE == "kernel" and packed_attention_supported(qkv, num_heads, max_len):
        return packed_attention(qkv, offsets, num_heads, max_len, p)
    if qkv.is_cuda and ATTENTION_MODE in ("padded", "kernel"):
        return _attention_padded(qkv, offsets, num_heads, max_len, p)
    q, k, v = (t.reshape(T, num_heads, D // num_heads) for t in qkv.split(D, dim=1))
    if qkv.is_cuda:
        jag = offsets.to(torch.int64)
        parts = [torch.nested.nested_tensor_from_jagged(t.contiguous(), offsets=jag, min_seqlen=0, max_seqlen=int(max_len)).transpose(1, 2) for t in (q, k, v)]
        out = torch.nn.functional.scaled_dot_product_attention(parts[0], parts[1], parts[2], dropout_p=p)
        return out.transpose(1, 2).values().reshape(T, D)
    return _attention_per_sequence(q, k, v, offsets, p).reshape(T, D)


def jagged_encoder_forward(encoder: nn.TransformerEncoder, x: torch.Tensor, offsets: torch.Tensor, max_len: int,
                           training: Optional[bool] = None) -> torch.Tensor:
    """``x [T, D]`` packed tokens, ``offsets [B + 1]`` sequence bounds; returns the encoded tokens ``[T, D]`` in ``x``'s dtype
    (bf16 inside when the fused dense path is on)."""
    training = encoder.training if training is None else training
    fused = dense_ops.fused_dense_enabled(x)
    T = x.shape[0]
    s = x.to(torch.bfloat16) if fused else x
    pad = (-T) % 8 if fused else 0
    if pad:  # the weight-gradient GEMMs want a token count that is a multiple of 8: a short dummy sequence at the end
        s = torch.cat([s, s.new_zeros(pad, s.shape[1])])
        offsets = torch.cat([offsets, offsets.new_tensor([T + pad])])
    s = s.contiguous()
    pending: Optional[torch.Tensor] = None  # output of the previous sub-block, not yet added to the stream
    pending_p = 0.0
    with torch.autocast(device_type=x.device.type, enabled=False):
        for layer in encoder.layers:
            attn = layer.self_attn
            # (dropout + add of the previous feed-forward output) + norm1, in one pass
            s, y = residual_layer_norm(pending, s, layer.norm1.weight, layer.norm1.bias, pending_p, training, layer.norm1.eps)
            qkv = dense_ops.linear_act(y, attn.in_proj_weight, attn.in_proj_bias)
            ctx = varlen_attention(qkv, offsets, attn.num_heads, max_len, attn.dropout if training else 0.0)
            o = dense_ops.linear_act(ctx, attn.out_proj.weight, attn.out_proj.bias)
            s, y = residual_layer_norm(o, s, layer.norm2.weight, layer.norm2.bias, layer.dropout1.p, training, layer.norm2.eps)
            h = gelu_dropout(dense_ops.linear_act(y, layer.linear1.weight, layer.linear1.bias), layer.dropout.p, training)
            pending = dense_ops.linear_act(h, layer.linear2.weight, layer.linear2.bias)
            pending_p = layer.dropout2.p
        if encoder.norm is not None:
            s, out = residual_layer_norm(pending, s, encoder.norm.weight, encoder.norm.bias, pending_p, training, encoder.norm.eps)
        else:
            out = s + torch.nn.functional.dropout(pending, pending_p, training=training and pending_p > 0)
    return out[:T] if pad else out
