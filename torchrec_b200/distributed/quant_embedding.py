"""Sharded quantized ``EmbeddingCollection`` (sequence embeddings) for single-process multi-device inference; table-wise
placement, synchronous forward returning ``Dict[feature, JaggedTensor]`` (cf. ``torchrec/distributed/quant_embedding.py:549``)."""
from __future__ import annotations

import copy
from typing import Any, Dict, List, Optional, Type

import torch
from torch import nn

from torchrec_b200.distributed.embedding_types import BaseQuantEmbeddingSharder
from torchrec_b200.distributed.quant_embeddingbag import _device_for
from torchrec_b200.distributed.types import ParameterSharding, ShardingEnv, ShardingType
from torchrec_b200.quant.embedding_modules import EmbeddingCollection as QuantEmbeddingCollection
from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor


class ShardedQuantEmbeddingCollection(nn.Module):
    def __init__(self, module: QuantEmbeddingCollection, table_name_to_parameter_sharding: Dict[str, ParameterSharding], env: ShardingEnv,
                 fused_params: Optional[Dict[str, Any]] = None, device: Optional[torch.device] = None) -> None:
        super().__init__()
        self._configs = module.embedding_configs()
        self._world_size = env.world_size
        self._device_type = (device.type if device is not None else ("cuda" if torch.cuda.is_available() else "cpu"))
        self._out_device = device if device is not None else _device_for(0, self._device_type)
        by_rank: List[List[Any]] = [[] for _ in range(self._world_size)]
        for cfg in self._configs:
            ps = table_name_to_parameter_sharding[cfg.name]
            if ps.sharding_type != ShardingType.TABLE_WISE.value:
                raise ValueError(f"quantized inference sharding supports table_wise placement, got {ps.sharding_type} for {cfg.name}")
            by_rank[ps.ranks[0]].append(cfg)
        self._shards = nn.ModuleList()
        self._feature_names_per_rank: List[List[str]] = []
        for rank, cfgs in enumerate(by_rank):
            if not cfgs:
                self._shards.append(nn.Identity())
                self._feature_names_per_rank.append([])
                continue
            dev = _device_for(rank, self._device_type)
            shard = QuantEmbeddingCollection(copy.deepcopy(cfgs), dev, need_indices=module.need_indices(), output_dtype=module.output_dtype())
            for cfg in cfgs:
                shard.embeddings[cfg.name].weight.copy_(module.embeddings[cfg.name].weight.to(dev))
            # shared-feature names must match the unsharded module's (feature@table)
            shard._name_of = {k: v for k, v in module._name_of.items() if k.split(":")[0] in {c.name for c in cfgs}}
            self._shards.append(shard)
            self._feature_names_per_rank.append([f for c in cfgs for f in c.feature_names])

    def forward(self, features: KeyedJaggedTensor) -> Dict[str, JaggedTensor]:
        keys = features.keys()
        out: Dict[str, JaggedTensor] = {}
        for rank, (shard, fnames) in enumerate(zip(self._shards, self._feature_names_per_rank)):
            if not fnames:
                continue
            dev = _device_for(rank, self._device_type)
            local = features.permute([keys.index(f) for f in fnames]).to(dev, non_blocking=True)
            for k, jt in shard(local).items():
                out[k] = jt.to(self._out_device)
        return out


class QuantEmbeddingCollectionSharder(BaseQuantEmbeddingSharder[QuantEmbeddingCollection]):
    def shard(self, module: QuantEmbeddingCollection, params: Dict[str, ParameterSharding], env: ShardingEnv,
              device: Optional[torch.device] = None, module_fqn: Optional[str] = None) -> ShardedQuantEmbeddingCollection:
        return ShardedQuantEmbeddingCollection(module, params, env, getattr(self, "fused_params", None), device)

    def shardable_parameters(self, module: QuantEmbeddingCollection) -> Dict[str, torch.Tensor]:
        return {name: m.weight for name, m in module.embeddings.items()}

    def sharding_types(self, compute_device_type: str) -> List[str]:
        return [ShardingType.TABLE_WISE.value]

    @property
    def module_type(self) -> Type[QuantEmbeddingCollection]:
        return QuantEmbeddingCollection
