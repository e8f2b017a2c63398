"""Row-wise N-bit quantization of embedding tables.

Row format: ``D * bits / 8`` payload bytes, then an fp16 scale and an fp16 bias (4 trailing bytes);
``value = scale * q + bias`` with ``q`` in ``[0, 2^bits - 1]``.  Same format as the reference's quantized state dict
(``torchrec/quant/embedding_modules.py:261-276``), so packed tables are interchangeable.
"""
from __future__ import annotations

from typing import Tuple

import torch

from torchrec_b200.modules.embedding_configs import DataType

BITS = {DataType.INT8: 8, DataType.INT4: 4, DataType.INT2: 2, DataType.FP16: 16, DataType.FP32: 32}


def row_bytes(dim: int, bits: int) -> int:
    return dim * bits // 8 + (4 if bits < 16 else 0)


def quantize_rowwise_nbit(weight: torch.Tensor, bits: int) -> torch.Tensor:
    """``[R, D]`` -> uint8 ``[R, row_bytes]`` (one kernel on a CUDA device: a warp per row finds min/max and packs)."""
    assert weight.dim() == 2
    R, D = weight.shape
    w = weight.detach().float()
    if bits == 32:
        return w.contiguous().view(torch.uint8).view(R, D * 4)
    if bits == 16:
        return w.half().contiguous().view(torch.uint8).view(R, D * 2)
    assert bits in (8, 4, 2) and (D * bits) % 8 == 0
    if weight.is_cuda and R > 0:
        from . import _ext

        _ext.require_cuda_ext("rowwise_quantize_nbit")
        src = weight.detach()
        if src.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            src = src.float()
        return torch.ops.trb200.rowwise_quantize_nbit(src.contiguous(), bits)
    qmax = float(2 ** bits - 1)
    lo = w.min(dim=1, keepdim=True).values if R else w.new_zeros(0, 1)
    hi = w.max(dim=1, keepdim=True).values if R else w.new_zeros(0, 1)
    # scale and bias are stored in fp16: quantize against the values the kernel will actually use
    scale = ((hi - lo) / qmax).half().float()
    scale = torch.where(scale == 0, torch.ones_like(scale), scale)
    bias = lo.half().float()
    q = torch.clamp(torch.round((w - bias) / scale), 0, qmax).to(torch.uint8)
    if bits == 8:
        payload = q
    else:
        per = 8 // bits
        q = q.view(R, D // per, per).to(torch.int32)
        shifts = torch.arange(per, device=w.device, dtype=torch.int32) * bits
        payload = (q << shifts).sum(dim=-1).to(torch.uint8)
    tail = torch.stack([scale.squeeze(1).half(), bias.squeeze(1).half()], dim=1).contiguous().view(torch.uint8).view(R, 4)
    return torch.cat([payload, tail], dim=1).contiguous()


def dequantize_rowwise_nbit(packed: torch.Tensor, dim: int, bits: int) -> torch.Tensor:
    """uint8 ``[R, row_bytes]`` -> fp32 ``[R, D]``."""
    R = packed.shape[0]
    if bits == 32:
        return packed.contiguous().view(torch.float32).view(R, dim).clone()
    if bits == 16:
        return packed.contiguous().view(torch.float16).view(R, dim).float()
    nb = dim * bits // 8
    payload = packed[:, :nb]
    tail = packed[:, nb: nb + 4].contiguous().view(torch.float16).view(R, 2).float()
    scale, bias = tail[:, :1], tail[:, 1:]
    if bits == 8:
        q = payload.float()
    else:
        per = 8 // bits
        shifts = torch.arange(per, device=packed.device, dtype=torch.int32) * bits
        q = ((payload.to(torch.int32).unsqueeze(-1) >> shifts) & (2 ** bits - 1)).reshape(R, dim).float()
    return q * scale + bias


def split_scale_bias(packed: torch.Tensor, dim: int, bits: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(payload [R, D*bits/8] uint8, scale_bias [R, 2] fp16)`` views of a packed table."""
    nb = dim * bits // 8
    return packed[:, :nb], packed[:, nb: nb + 4].contiguous().view(torch.float16).view(-1, 2)
