"""Sharders of the single-device fused collections: a ``FusedEmbeddingBagCollection`` / ``FusedEmbeddingCollection`` carries its
optimizer with it, so sharding it means sharding a plain collection of the same tables with that optimizer fused into the lookup
kernels, and moving the weights over.  Counterpart of ``torchrec/distributed/fused_embeddingbag.py:34`` and ``fused_embedding.py:31``."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Type

import torch
from torch import nn

from torchrec_b200.distributed.embedding import EmbeddingCollectionSharder, ShardedEmbeddingCollection
from torchrec_b200.distributed.embedding_types import BaseEmbeddingSharder, EmbeddingComputeKernel
from torchrec_b200.distributed.embeddingbag import EmbeddingBagCollectionSharder, ShardedEmbeddingBagCollection
from torchrec_b200.distributed.types import ParameterSharding, QuantizedCommCodecs, ShardingEnv, ShardingType
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection, EmbeddingCollection
from torchrec_b200.modules.fused_embedding_modules import FusedEmbeddingBagCollection, FusedEmbeddingCollection
from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward


class ShardedFusedEmbeddingBagCollection(ShardedEmbeddingBagCollection):
    @property
    def unsharded_module_type(self) -> Type[FusedEmbeddingBagCollection]:
        return FusedEmbeddingBagCollection


class ShardedFusedEmbeddingCollection(ShardedEmbeddingCollection):
    @property
    def unsharded_module_type(self) -> Type[FusedEmbeddingCollection]:
        return FusedEmbeddingCollection


@torch.no_grad()
def _copy_weights(fused: nn.Module, sharded: nn.Module, container: str) -> None:
    src = getattr(fused, container)
    if any(m.weight.device.type == "meta" for m in src.values()):
        return
    for name, shards in sharded._model_parallel_name_to_local_shards.items():
        full = src[name].weight
        for t, w in shards:
            ro, co = t.local_metadata.shard_offsets
            rs, cs = t.local_metadata.shard_sizes
            w.copy_(full[ro:ro + rs, co:co + cs].to(w.device))


class FusedEmbeddingBagCollectionSharder(BaseEmbeddingSharder[FusedEmbeddingBagCollection]):
    def shard(self, module: FusedEmbeddingBagCollection, params: Dict[str, ParameterSharding], env: ShardingEnv, device: Optional[torch.device] = None,
              module_fqn: Optional[str] = None) -> ShardedFusedEmbeddingBagCollection:
        stub = EmbeddingBagCollection(tables=module.embedding_bag_configs(), is_weighted=module.is_weighted(), device=torch.device("meta"))
        apply_optimizer_in_backward(module._optimizer_type, stub.parameters(), dict(module._optimizer_kwargs))
        sharded = ShardedFusedEmbeddingBagCollection(stub, params, env, fused_params=self.fused_params, device=device, qcomm_codecs_registry=self.qcomm_codecs_registry,
                                                     module_fqn=module_fqn)
        _copy_weights(module, sharded, "embedding_bags")
        return sharded

    def shardable_parameters(self, module: FusedEmbeddingBagCollection) -> Dict[str, nn.Parameter]:
        return {name: m.weight for name, m in module.embedding_bags.items()}

    @property
    def module_type(self) -> Type[FusedEmbeddingBagCollection]:
        return FusedEmbeddingBagCollection

    def sharding_types(self, compute_device_type: str) -> List[str]:
        return [t for t in super().sharding_types(compute_device_type) if t != ShardingType.DATA_PARALLEL.value]

    def compute_kernels(self, sharding_type: str, compute_device_type: str) -> List[str]:
        return [k for k in super().compute_kernels(sharding_type, compute_device_type) if k != EmbeddingComputeKernel.DENSE.value]


class FusedEmbeddingCollectionSharder(BaseEmbeddingSharder[FusedEmbeddingCollection]):
    def shard(self, module: FusedEmbeddingCollection, params: Dict[str, ParameterSharding], env: ShardingEnv, device: Optional[torch.device] = None,
              module_fqn: Optional[str] = None) -> ShardedFusedEmbeddingCollection:
        stub = EmbeddingCollection(tables=module.embedding_configs(), device=torch.device("meta"), need_indices=module.need_indices())
        apply_optimizer_in_backward(module._optimizer_type, stub.parameters(), dict(module._optimizer_kwargs))
        sharded = ShardedFusedEmbeddingCollection(stub, params, env, fused_params=self.fused_params, device=device, qcomm_codecs_registry=self.qcomm_codecs_registry,
                                                  module_fqn=module_fqn)
        _copy_weights(module, sharded, "embeddings")
        return sharded

    def shardable_parameters(self, module: FusedEmbeddingCollection) -> Dict[str, nn.Parameter]:
        return {name: m.weight for name, m in module.embeddings.items()}

    @property
    def module_type(self) -> Type[FusedEmbeddingCollection]:
        return FusedEmbeddingCollection

    def sharding_types(self, compute_device_type: str) -> List[str]:
        return [ShardingType.TABLE_WISE.value, ShardingType.COLUMN_WISE.value, ShardingType.ROW_WISE.value]

    def compute_kernels(self, sharding_type: str, compute_device_type: str) -> List[str]:
        return [k for k in super().compute_kernels(sharding_type, compute_device_type) if k != EmbeddingComputeKernel.DENSE.value]
