"""Shard-level quantized lookup kernels: the tables one device holds of one group, batched into one quantized lookup.

``QuantBatchedEmbeddingBag`` (pooled) and ``QuantBatchedEmbedding`` (sequence) are built from a ``GroupedEmbeddingConfig`` (local rows
and columns of every table shard) or, with ``from_float``, from a float shard kernel whose weights they quantize row-wise.
Counterpart of ``torchrec/distributed/quant_embedding_kernel.py:228-620``."""
from __future__ import annotations

from typing import Any, Dict, Iterator, List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import nn

from torchrec_b200.distributed.embedding_types import GroupedEmbeddingConfig
from torchrec_b200.distributed.fused_params import TBEToRegisterMixIn, get_fused_param_tbe_row_alignment, tbe_fused_params
from torchrec_b200.modules.embedding_configs import DataType, pooling_type_to_pooling_mode
from torchrec_b200.ops.qtbe import QuantTableBatchedEmbeddingBags
from torchrec_b200.ops.quant_ops import BITS, quantize_rowwise_nbit
from torchrec_b200.ops.tbe import PoolingMode
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


def _quantize_weight(weight: torch.Tensor, data_type: DataType) -> torch.Tensor:
    """Float ``[rows, dim]`` -> packed uint8 rows of ``data_type`` (payload, then fp16 scale and bias for sub-16-bit types)."""
    return quantize_rowwise_nbit(weight.detach().float(), BITS[data_type])


class _QuantBatchedBase(nn.Module, TBEToRegisterMixIn):
    _pooled: bool = True

    def __init__(self, config: GroupedEmbeddingConfig, pg: Optional[dist.ProcessGroup] = None, device: Optional[torch.device] = None,
                 fused_params: Optional[Dict[str, Any]] = None) -> None:
        super().__init__()
        self._config, self._pg = config, pg
        self._fused_params = tbe_fused_params(fused_params) or {}
        self._row_alignment = get_fused_param_tbe_row_alignment(fused_params)
        tables = config.embedding_tables
        specs = [(max(t.local_rows, 1), t.local_cols, BITS[config.data_type]) for t in tables]
        ftm = [i for i, t in enumerate(tables) for _ in t.feature_names]
        mode = pooling_type_to_pooling_mode(config.pooling) if self._pooled else PoolingMode.NONE
        out_dtype = self._fused_params.get("output_dtype", torch.float32)
        self._emb_module = QuantTableBatchedEmbeddingBags(specs, ftm, mode, out_dtype if isinstance(out_dtype, torch.dtype) else torch.float32,
                                                          device=device if device is not None and device.type != "meta" else None)
        self._feature_names = config.feature_names()

    @property
    def emb_module(self) -> QuantTableBatchedEmbeddingBags:
        return self._emb_module

    @property
    def config(self) -> GroupedEmbeddingConfig:
        return self._config

    def get_tbes_to_register(self) -> Dict[nn.Module, GroupedEmbeddingConfig]:
        return {self._emb_module: self._config}

    def split_embedding_weights(self) -> List[torch.Tensor]:
        return self._emb_module.split_embedding_weights()

    def named_buffers(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True) -> Iterator[Tuple[str, torch.Tensor]]:
        for t, w in zip(self._config.embedding_tables, self.split_embedding_weights()):
            yield (f"{prefix}.{t.name}.weight" if prefix else f"{t.name}.weight"), w

    def named_parameters(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True) -> Iterator[Tuple[str, nn.Parameter]]:
        yield from ()

    def forward(self, features: KeyedJaggedTensor) -> torch.Tensor:
        weights = features.weights_or_none() if self._pooled and self._config.is_weighted else None
        return self._emb_module(features.values(), features.offsets(), weights)

    @classmethod
    def from_float(cls, module: nn.Module, use_precomputed_fake_quant: bool = False, data_type: DataType = DataType.INT8):
        """Quantize the shard weights of a float kernel (anything with ``config`` and ``split_embedding_weights()``)."""
        import copy

        config = copy.deepcopy(module.config)
        config.data_type = data_type
        for t in config.embedding_tables:
            t.data_type = data_type
        floats = module.split_embedding_weights()
        device = floats[0].device if floats else torch.device("cpu")
        out = cls(config, device=device)
        for dst, src, t in zip(out.split_embedding_weights(), floats, config.embedding_tables):
            if t.local_rows > 0:
                dst.copy_(_quantize_weight(src.reshape(t.local_rows, t.local_cols), data_type).to(dst.device))
        return out


class QuantBatchedEmbeddingBag(_QuantBatchedBase):
    """``forward(KJT of this group's features) -> [B, sum(local dims)]``."""

    _pooled = True


class QuantBatchedEmbedding(_QuantBatchedBase):
    """``forward(KJT of this group's features) -> [num ids, local dim]``."""

    _pooled = False
