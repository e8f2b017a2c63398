"""Quantized-communication codecs: cast (or row-wise quantise) embedding payloads around a collective.

``QCommsConfig`` picks a forward and a backward precision per collective; ``get_qcomm_codecs_registry``
builds the ``{CommOp name: QuantizedCommCodecs}`` map the sharders consume.  The file keeps the name the
reference uses (``torchrec/distributed/fbgemm_qcomm_codec.py:32-234``) so that user imports carry over;
the codecs themselves are implemented here.  On the fused NVLink paths the cast happens inside the
lookup / gradient kernels and these standalone codecs are bypassed.
"""
from __future__ import annotations

import copy
import logging
from dataclasses import dataclass
from enum import Enum, unique
from typing import Any, Dict, List, Optional, Tuple, cast

import torch

from torchrec_b200.distributed.types import CommOp, QuantizedCommCodec, QuantizedCommCodecs

logger: logging.Logger = logging.getLogger()


@unique
class CommType(Enum):
    FP32 = "fp32"
    FP16 = "fp16"
    BF16 = "bf16"
    FP8 = "fp8"
    INT8 = "int8"
    MX4 = "mx4"

    def __str__(self) -> str:
        return self.value


def comm_type_to_sparse_type(comm_type: CommType) -> "SparseType":
    """The kernel-side element type of a wire precision.  MX4 (4-bit values with shared block exponents) has no element type of
    its own in this package's kernels: its payload is carried as packed 4-bit codes."""
    from torchrec_b200.modules.embedding_configs import SparseType

    return {CommType.FP32: SparseType.FP32, CommType.FP16: SparseType.FP16, CommType.BF16: SparseType.BF16, CommType.FP8: SparseType.FP8,
            CommType.INT8: SparseType.INT8, CommType.MX4: SparseType.INT4}[comm_type]


def comm_type_to_dtype(comm_type: CommType) -> torch.dtype:
    return {
        CommType.FP32: torch.float32, CommType.FP16: torch.float16, CommType.BF16: torch.bfloat16,
        CommType.FP8: torch.uint8, CommType.INT8: torch.uint8, CommType.MX4: torch.uint8,
    }[comm_type]


@dataclass
class QCommsConfig:
    """Forward / backward precision of the embedding collectives (typical: FP16 forward, BF16 backward)."""

    forward_precision: CommType = CommType.FP32
    backward_precision: CommType = CommType.FP32
    forward_loss_scale: Optional[float] = None
    backward_loss_scale: Optional[float] = None
    fp8_quantize_dim: Optional[int] = None
    fp8_quantize_dim_bwd: Optional[int] = None
    fp8_bwd_uses_143: Optional[bool] = False
    mx4_quantize_dim: Optional[int] = None
    mx4_quantize_dim_bwd: Optional[int] = None
    mx4_rounding_mode: Optional[Any] = None

    def __post_init__(self) -> None:
        if self.forward_precision != CommType.FP8 and self.backward_precision != CommType.FP8 and (
            self.fp8_quantize_dim is not None or self.fp8_quantize_dim_bwd is not None
        ):
            raise ValueError(
                f"fp8_quantize_dim is set to {self.fp8_quantize_dim} and fp8_quantize_dim_bwd is set to {self.fp8_quantize_dim_bwd} "
                "but no FP8 precision is found in forward or backward precisions"
            )
        if self.backward_precision == CommType.FP8 and self.fp8_quantize_dim_bwd is None:
            self.fp8_quantize_dim_bwd = self.fp8_quantize_dim
            logger.warning(f"No override of FP8 bwd row dim, using general FP8 row dim for backward: {self.fp8_quantize_dim_bwd}")


class _Ctx:
    def __init__(self, row_dim: int = -1) -> None:
        self.row_dim = row_dim
        self.shape: Optional[torch.Size] = None
        self.dtype: Optional[torch.dtype] = None


class CastCodec(QuantizedCommCodec):
    """fp32 <-> fp16 / bf16 cast with an optional loss scale."""

    def __init__(self, comm_type: CommType, loss_scale: Optional[float] = None, is_fwd: bool = True) -> None:
        self._comm_type = comm_type
        self._dtype = comm_type_to_dtype(comm_type)
        self._loss_scale = loss_scale
        self._is_fwd = is_fwd

    def encode(self, input_tensor: torch.Tensor, ctx: Optional[_Ctx] = None) -> torch.Tensor:
        if ctx is not None:
            ctx.dtype = input_tensor.dtype
        if self._comm_type == CommType.FP32:
            return input_tensor
        t = input_tensor
        if self._loss_scale is not None:
            t = t * self._loss_scale
        return t.to(self._dtype)

    def decode(self, input_grad: torch.Tensor, ctx: Optional[_Ctx] = None) -> torch.Tensor:
        if self._comm_type == CommType.FP32:
            return input_grad
        out_dtype = ctx.dtype if ctx is not None and ctx.dtype is not None else torch.float32
        t = input_grad.to(out_dtype)
        if self._loss_scale is not None:
            t = t / self._loss_scale
        return t

    @property
    def quantized_dtype(self) -> torch.dtype:
        return self._dtype

    def calc_quantized_size(self, input_len: int, ctx: Optional[_Ctx] = None) -> int:
        return input_len

    def create_context(self) -> Optional[_Ctx]:
        return _Ctx()


class RowwiseInt8Codec(QuantizedCommCodec):
    """Row-wise 8-bit quantisation: every ``row_dim`` values share an fp32 scale and bias appended to the
    row (``row_dim + 8`` bytes per row).  Used for ``CommType.INT8`` and as the container of ``FP8``
    (scaled e4m3 stored in a byte)."""

    def __init__(self, comm_type: CommType, row_dim: Optional[int] = None, is_fwd: bool = True) -> None:
        self._comm_type = comm_type
        self._row_dim = row_dim if row_dim and row_dim > 0 else -1
        self._is_fwd = is_fwd

    def _rows(self, numel: int) -> Tuple[int, int]:
        rd = self._row_dim if self._row_dim > 0 else numel
        assert numel % rd == 0, f"payload of {numel} elements is not a multiple of the quantisation row {rd}"
        return numel // rd, rd

    def encode(self, input_tensor: torch.Tensor, ctx: Optional[_Ctx] = None) -> torch.Tensor:
        flat = input_tensor.reshape(-1).float()
        if ctx is not None and ctx.row_dim > 0 and self._row_dim <= 0 and flat.numel() % ctx.row_dim == 0:
            n, rd = flat.numel() // ctx.row_dim, ctx.row_dim  # the caller knows the row width of this chunk
        else:
            n, rd = self._rows(flat.numel())
        x = flat.view(n, rd)
        if ctx is not None:
            ctx.dtype = input_tensor.dtype
            ctx.row_dim = rd
        if self._comm_type == CommType.FP8:
            amax = x.abs().amax(dim=1, keepdim=True).clamp(min=1e-12)
            scale = 448.0 / amax
            q = (x * scale).to(torch.float8_e4m3fn).view(torch.uint8)
            meta = torch.cat([scale, torch.zeros_like(scale)], dim=1)
        else:
            mn = x.amin(dim=1, keepdim=True)
            mx = x.amax(dim=1, keepdim=True)
            scale = ((mx - mn) / 255.0).clamp(min=1e-12)
            q = torch.round((x - mn) / scale).clamp(0, 255).to(torch.uint8)
            meta = torch.cat([scale, mn], dim=1)
        return torch.cat([q, meta.contiguous().view(torch.uint8).view(n, 8)], dim=1).reshape(-1)

    def decode(self, input_grad: torch.Tensor, ctx: Optional[_Ctx] = None) -> torch.Tensor:
        rd = ctx.row_dim if ctx is not None and ctx.row_dim > 0 else self._row_dim
        assert rd > 0, "row dim unknown: decode needs the context created for encode"
        x = input_grad.view(-1, rd + 8)
        q = x[:, :rd]
        meta = x[:, rd:].contiguous().view(torch.float32).view(-1, 2)
        if self._comm_type == CommType.FP8:
            out = q.contiguous().view(torch.float8_e4m3fn).float() / meta[:, :1]
        else:
            out = q.float() * meta[:, :1] + meta[:, 1:2]
        out_dtype = ctx.dtype if ctx is not None and ctx.dtype is not None else torch.float32
        return out.reshape(-1).to(out_dtype)

    @property
    def quantized_dtype(self) -> torch.dtype:
        return torch.uint8

    def calc_quantized_size(self, input_len: int, ctx: Optional[_Ctx] = None) -> int:
        rd = ctx.row_dim if ctx is not None and ctx.row_dim > 0 else self._row_dim
        if rd <= 0:
            return input_len + 8
        assert input_len % rd == 0
        return input_len // rd * (rd + 8)

    def create_context(self) -> Optional[_Ctx]:
        return _Ctx(self._row_dim)

    def padded_size(self, input_tensor: torch.Tensor, dim_per_rank: List[int], my_rank: int, qcomm_ctx: _Ctx) -> Tuple[int, int]:
        if input_tensor.ndim == 1:
            return input_tensor.shape[0], 0
        dim_sum = input_tensor.shape[1]
        rd = qcomm_ctx.row_dim
        if rd > 0 and dim_sum % rd != 0:
            padded = (dim_sum + rd - 1) // rd * rd
            return padded, padded - dim_sum
        return dim_sum, 0


class Mx4Codec(QuantizedCommCodec):
    """Microscaling 4-bit format: blocks of ``group`` values (default 32) share one power-of-two scale stored as a biased
    8-bit exponent, every value is a 4-bit e2m1 float (sign, magnitudes 0 / 0.5 / 1 / 1.5 / 2 / 3 / 4 / 6), two per byte:
    ``group / 2 + 1`` bytes per block, 4.25 bits per value at group 32.  The payload is padded to whole blocks."""

    _LEVELS = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)

    def __init__(self, group: Optional[int] = None, is_fwd: bool = True) -> None:
        self._group = int(group) if group and group > 0 else 32
        assert self._group % 2 == 0, "two 4-bit codes share a byte"
        self._is_fwd = is_fwd

    def encode(self, input_tensor: torch.Tensor, ctx: Optional[_Ctx] = None) -> torch.Tensor:
        g = self._group
        flat = input_tensor.reshape(-1).float()
        if ctx is not None:
            ctx.dtype = input_tensor.dtype
            ctx.numel = flat.numel()
        pad = (-flat.numel()) % g
        if pad:
            flat = torch.cat([flat, flat.new_zeros(pad)])
        x = flat.view(-1, g)
        amax = x.abs().amax(dim=1, keepdim=True)
        # largest magnitude maps into (4, 6]: shared exponent = floor(log2(amax)) - 2, kept in [-127, 127]
        exp = torch.where(amax > 0, torch.floor(torch.log2(amax.clamp(min=1e-38))) - 2, torch.full_like(amax, -127.0)).clamp(-127, 127)
        y = x / torch.exp2(exp)
        levels = torch.tensor(self._LEVELS, device=x.device)
        mag = (y.abs().unsqueeze(-1) - levels).abs().argmin(dim=-1)  # nearest representable magnitude (saturates at 6)
        code = (mag | ((y < 0).to(torch.int64) << 3)).to(torch.uint8)
        packed = code[:, 0::2] | (code[:, 1::2] << 4)
        return torch.cat([packed, (exp + 127).to(torch.uint8)], dim=1).reshape(-1)

    def decode(self, input_grad: torch.Tensor, ctx: Optional[_Ctx] = None) -> torch.Tensor:
        g = self._group
        blocks = input_grad.view(-1, g // 2 + 1)
        packed, exp = blocks[:, : g // 2], blocks[:, g // 2:].float() - 127
        code = torch.stack([packed & 0xF, packed >> 4], dim=2).reshape(-1, g).long()
        levels = torch.tensor(self._LEVELS, device=input_grad.device)
        val = levels[code & 7] * torch.where((code & 8) != 0, -1.0, 1.0) * torch.exp2(exp)
        out = val.reshape(-1)
        n = getattr(ctx, "numel", None) if ctx is not None else None
        if n is not None:
            out = out[:n]
        out_dtype = ctx.dtype if ctx is not None and ctx.dtype is not None else torch.float32
        return out.to(out_dtype)

    @property
    def quantized_dtype(self) -> torch.dtype:
        return torch.uint8

    def calc_quantized_size(self, input_len: int, ctx: Optional[_Ctx] = None) -> int:
        g = self._group
        return (input_len + g - 1) // g * (g // 2 + 1)

    def create_context(self) -> Optional[_Ctx]:
        return _Ctx(self._group)

    def padded_size(self, input_tensor: torch.Tensor, dim_per_rank: List[int], my_rank: int, qcomm_ctx: _Ctx) -> Tuple[int, int]:
        if input_tensor.ndim == 1:
            return input_tensor.shape[0], 0
        width, g = input_tensor.shape[1], self._group
        padded = (width + g - 1) // g * g
        return padded, padded - width


def get_qcomm_codecs(qcomms_config: Optional[QCommsConfig]) -> QuantizedCommCodecs:
    codecs = QuantizedCommCodecs()
    if qcomms_config is not None:
        def make(comm_type: CommType, loss_scale, row_dim, is_fwd: bool) -> QuantizedCommCodec:
            if comm_type in (CommType.FP32, CommType.FP16, CommType.BF16):
                return CastCodec(comm_type, loss_scale, is_fwd)
            if comm_type == CommType.MX4:
                return Mx4Codec(row_dim, is_fwd)
            return RowwiseInt8Codec(comm_type, row_dim, is_fwd)

        fwd_dim = qcomms_config.fp8_quantize_dim if qcomms_config.forward_precision == CommType.FP8 else qcomms_config.mx4_quantize_dim
        bwd_dim = qcomms_config.fp8_quantize_dim_bwd if qcomms_config.backward_precision == CommType.FP8 else qcomms_config.mx4_quantize_dim_bwd
        codecs.forward = make(qcomms_config.forward_precision, qcomms_config.forward_loss_scale, fwd_dim, True)
        codecs.backward = make(qcomms_config.backward_precision, qcomms_config.backward_loss_scale, bwd_dim, False)
    return codecs


def get_qcomm_codecs_registry(qcomms_config: QCommsConfig, comm_ops: Optional[List[CommOp]] = None, device: Optional[torch.device] = None) -> Optional[Dict[str, QuantizedCommCodecs]]:
    """``{CommOp.name: codecs}`` for the given ops (default: all).  Reduce-scatter sums on the wire, so
    byte-quantised formats fall back to FP16 (forward) / BF16 (backward) there; on CPU (gloo) BF16 becomes FP16."""
    if qcomms_config.forward_precision == CommType.FP32 and qcomms_config.backward_precision == CommType.FP32:
        return None
    if device is not None and device.type == "cpu":
        return None
    if comm_ops is None:
        comm_ops = [CommOp.POOLED_EMBEDDINGS_ALL_TO_ALL, CommOp.POOLED_EMBEDDINGS_REDUCE_SCATTER, CommOp.SEQUENCE_EMBEDDINGS_ALL_TO_ALL]
    registry: Dict[str, QuantizedCommCodecs] = {}
    for comm_op in comm_ops:
        cfg = qcomms_config
        if comm_op == CommOp.POOLED_EMBEDDINGS_REDUCE_SCATTER:
            byte_formats = (CommType.FP8, CommType.INT8, CommType.MX4)
            if cfg.forward_precision in byte_formats or cfg.backward_precision in byte_formats:
                cfg = copy.deepcopy(cfg)
                if cfg.forward_precision in byte_formats:
                    logger.warning("byte-quantised forward precision is not supported for reduce-scatter; using FP16")
                    cfg.forward_precision = CommType.FP16
                if cfg.backward_precision in byte_formats:
                    logger.warning("byte-quantised backward precision is not supported for reduce-scatter; using BF16")
                    cfg.backward_precision = CommType.BF16
        registry[comm_op.name] = get_qcomm_codecs(cfg)
    return registry
