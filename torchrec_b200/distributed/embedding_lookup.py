"""Lookups of one rank: the TBE groups of a sharding, fed from one KJT.

``GroupedPooledEmbeddingsLookup`` (pooled, output ``[B, sum(D)]``) and ``GroupedEmbeddingsLookup``
(unpooled, output ``[sum(L), D]``) split the incoming KJT by TBE group, run each group's kernel and
concatenate.  Counterpart of ``torchrec/distributed/embedding_lookup.py:178-711``.
"""
from __future__ import annotations

from typing import Any, Dict, Iterator, List, Optional, Tuple, Union

import torch
import torch.distributed as dist
from torch import nn
from torch.autograd.function import FunctionCtx
from torch.nn.parallel import DistributedDataParallel

from torchrec_b200.distributed.batched_embedding_kernel import (
    BaseEmbedding,
    BatchedDenseEmbedding,
    BatchedDenseEmbeddingBag,
    BatchedFusedEmbedding,
    BatchedFusedEmbeddingBag,
)
from torchrec_b200.distributed.embedding_types import (
    BaseEmbeddingLookup,
    BaseGroupedFeatureProcessor,
    EmbeddingComputeKernel,
    GroupedEmbeddingConfig,
)
from torchrec_b200.distributed.types import ShardedTensor, ShardingType
from torchrec_b200.optim.fused import FusedOptimizerModule
from torchrec_b200.optim.keyed import CombinedOptimizer, KeyedOptimizer
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


def _load_state_dict(emb_modules: "nn.ModuleList", state_dict: Dict[str, Any]) -> Tuple[List[str], List[str]]:
    """Copy checkpoint shards into the local table views, matching shards by their offsets."""
    missing_keys: List[str] = []
    unexpected_keys = list(state_dict.keys())
    for emb_module in emb_modules:
        for key, dst_param in emb_module.state_dict().items():
            if key in state_dict:
                src_param = state_dict[key]
                if isinstance(dst_param, ShardedTensor):
                    assert isinstance(src_param, ShardedTensor)
                    assert len(dst_param.local_shards()) == len(src_param.local_shards())
                    for dst_shard, src_shard in zip(dst_param.local_shards(), src_param.local_shards()):
                        assert dst_shard.metadata.shard_offsets == src_shard.metadata.shard_offsets
                        assert dst_shard.metadata.shard_sizes == src_shard.metadata.shard_sizes
                        dst_shard.tensor.detach().copy_(src_shard.tensor)
                elif isinstance(src_param, ShardedTensor):
                    dst_param.detach().copy_(src_param.local_shards()[0].tensor)
                else:
                    assert isinstance(src_param, torch.Tensor) and isinstance(dst_param, torch.Tensor)
                    dst_param.detach().copy_(src_param)
                unexpected_keys.remove(key)
            else:
                missing_keys.append(key)
    return missing_keys, unexpected_keys


class CommOpGradientScaling(torch.autograd.Function):
    """Identity in forward, scales the gradient in backward (weighted features with gradient division)."""

    @staticmethod
    def forward(ctx: FunctionCtx, input_tensor: torch.Tensor, scale_gradient_factor: int) -> torch.Tensor:
        ctx.scale_gradient_factor = scale_gradient_factor
        return input_tensor

    @staticmethod
    def backward(ctx: FunctionCtx, grad_output: torch.Tensor):
        grad_output.mul_(ctx.scale_gradient_factor)
        return grad_output, None


class _GroupedLookupBase(BaseEmbeddingLookup[KeyedJaggedTensor, torch.Tensor]):
    def __init__(self) -> None:
        super().__init__()
        self._emb_modules: nn.ModuleList = nn.ModuleList()
        self._feature_splits: List[int] = []
        self.grouped_configs: List[GroupedEmbeddingConfig] = []

    def _finish_init(self, device: Optional[torch.device]) -> None:
        self.register_buffer("_dummy_embs_tensor", torch.empty([0], dtype=torch.float32, device=device, requires_grad=True), persistent=False)

    @property
    def emb_modules(self) -> nn.ModuleList:
        return self._emb_modules

    def state_dict(self, destination=None, prefix: str = "", keep_vars: bool = False) -> Dict[str, Any]:
        if destination is None:
            destination = {}
        for emb_module in self._emb_modules:
            emb_module.state_dict(destination, prefix, keep_vars)
        return destination

    def load_state_dict(self, state_dict, strict: bool = True):  # type: ignore[override]
        m, u = _load_state_dict(self._emb_modules, state_dict)
        return torch.nn.modules.module._IncompatibleKeys(missing_keys=m, unexpected_keys=u)

    def named_parameters(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True) -> Iterator[Tuple[str, nn.Parameter]]:
        for emb_module in self._emb_modules:
            yield from emb_module.named_parameters(prefix, recurse)

    def named_buffers(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True) -> Iterator[Tuple[str, torch.Tensor]]:
        for emb_module in self._emb_modules:
            yield from emb_module.named_buffers(prefix, recurse)

    def named_parameters_by_table(self) -> Iterator[Tuple[str, torch.Tensor]]:
        for emb_module in self._emb_modules:
            for cfg, w in zip(emb_module.config.embedding_tables, emb_module.split_embedding_weights()):
                yield cfg.name, w

    def prefetch(self, sparse_features: KeyedJaggedTensor, forward_stream=None) -> None:
        # every table is resident in HBM: nothing to stage
        return None

    def flush(self) -> None:
        for m in self._emb_modules:
            m.flush()

    def purge(self) -> None:
        for m in self._emb_modules:
            m.purge()


class GroupedEmbeddingsLookup(_GroupedLookupBase):
    """Unpooled lookup over the TBE groups of one rank -> ``[sum L, D]``."""

    def __init__(self, grouped_configs: List[GroupedEmbeddingConfig], pg: Optional[dist.ProcessGroup] = None, device: Optional[torch.device] = None) -> None:
        super().__init__()
        self.grouped_configs = grouped_configs
        for config in grouped_configs:
            self._emb_modules.append(self._create_embedding_kernel(config, pg, device))
            self._feature_splits.append(config.num_features())
        self._need_prefetch = False
        self._finish_init(device)

    @staticmethod
    def _create_embedding_kernel(config: GroupedEmbeddingConfig, pg, device) -> BaseEmbedding:
        if config.compute_kernel == EmbeddingComputeKernel.DENSE:
            return BatchedDenseEmbedding(config=config, pg=pg, device=device)
        if config.compute_kernel in (EmbeddingComputeKernel.FUSED, EmbeddingComputeKernel.FUSED_UVM, EmbeddingComputeKernel.FUSED_UVM_CACHING):
            return BatchedFusedEmbedding(config=config, pg=pg, device=device)
        raise ValueError(f"Compute kernel not supported {config.compute_kernel}")

    def forward(self, sparse_features: KeyedJaggedTensor) -> torch.Tensor:
        embeddings: List[torch.Tensor] = []
        features_by_group = sparse_features.split(self._feature_splits) if len(self._emb_modules) > 1 else [sparse_features]
        for emb_op, features in zip(self._emb_modules, features_by_group):
            embeddings.append(emb_op(features).view(-1))
        if len(embeddings) == 0:
            return self._dummy_embs_tensor
        dim = self._emb_modules[0].emb_module.max_D
        if len(embeddings) == 1:
            return embeddings[0].view(-1, dim)
        return torch.cat(embeddings).view(-1, dim)


class GroupedPooledEmbeddingsLookup(_GroupedLookupBase):
    """Pooled lookup over the TBE groups of one rank -> ``[B, sum(D)]``."""

    def __init__(self, grouped_configs: List[GroupedEmbeddingConfig], device: Optional[torch.device] = None, pg: Optional[dist.ProcessGroup] = None,
                 feature_processor: Optional[BaseGroupedFeatureProcessor] = None, scale_weight_gradients: bool = True,
                 sharding_type: Optional[ShardingType] = None) -> None:
        super().__init__()
        self.grouped_configs = grouped_configs
        self._sharding_type = sharding_type
        for config in grouped_configs:
            self._emb_modules.append(self._create_embedding_kernel(config, device, pg, sharding_type))
            self._feature_splits.append(config.num_features())
        self._feature_processor = feature_processor
        self._world_size: int = dist.get_world_size(pg) if pg is not None else 1
        self._scale_gradient_factor: int = self._world_size if scale_weight_gradients else 1
        self._finish_init(device)

    @staticmethod
    def _create_embedding_kernel(config: GroupedEmbeddingConfig, device, pg, sharding_type) -> BaseEmbedding:
        if config.compute_kernel == EmbeddingComputeKernel.DENSE:
            return BatchedDenseEmbeddingBag(config=config, pg=pg, device=device, sharding_type=sharding_type)
        if config.compute_kernel in (EmbeddingComputeKernel.FUSED, EmbeddingComputeKernel.FUSED_UVM, EmbeddingComputeKernel.FUSED_UVM_CACHING):
            return BatchedFusedEmbeddingBag(config=config, pg=pg, device=device, sharding_type=sharding_type)
        raise ValueError(f"Compute kernel not supported {config.compute_kernel}")

    def forward(self, sparse_features: KeyedJaggedTensor) -> torch.Tensor:
        if len(self._emb_modules) == 0:
            return self._dummy_embs_tensor.view(sparse_features.stride(), 0) if sparse_features.stride() else self._dummy_embs_tensor
        embeddings: List[torch.Tensor] = []
        features_by_group = sparse_features.split(self._feature_splits) if len(self._emb_modules) > 1 else [sparse_features]
        for config, emb_op, features in zip(self.grouped_configs, self._emb_modules, features_by_group):
            if config.has_feature_processor and self._feature_processor is not None and isinstance(self._feature_processor, BaseGroupedFeatureProcessor):
                features = self._feature_processor(features)
            if config.is_weighted and self._scale_gradient_factor != 1 and features.weights_or_none() is not None and features.weights().requires_grad:
                features._weights = CommOpGradientScaling.apply(features._weights, self._scale_gradient_factor)
            embeddings.append(emb_op(features))
        if len(embeddings) == 1:
            return embeddings[0]
        return torch.cat(embeddings, dim=1)


def fused_optimizer_of_lookups(lookups: List[nn.Module]) -> KeyedOptimizer:
    """``CombinedOptimizer`` over the fused optimizers of every TBE in ``lookups``."""
    optims: List[KeyedOptimizer] = []
    for lookup in lookups:
        while isinstance(lookup, DistributedDataParallel):
            lookup = lookup.module
        for m in getattr(lookup, "emb_modules", []):
            if isinstance(m, FusedOptimizerModule):
                optims.append(m.fused_optimizer)
    return CombinedOptimizer(optims)
