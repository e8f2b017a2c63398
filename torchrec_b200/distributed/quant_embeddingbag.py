"""Sharded quantized ``EmbeddingBagCollection`` for inference: ONE process drives all devices.

Tables are placed table-wise (whole table on one device) following the module sharding plan; the request KJT is split
by feature and copied to the owning devices, each device runs one quantized lookup, and the pooled outputs are
concatenated on the output device in the key order of the unsharded module.  Synchronous ``forward`` (no awaitables),
as serving code expects.  Counterpart of ``torchrec/distributed/quant_embeddingbag.py:165-470`` (table-wise path).
"""
from __future__ import annotations

import copy
from typing import Any, Dict, List, Optional, Type

import torch
from torch import nn

from torchrec_b200.distributed.embedding_types import BaseQuantEmbeddingSharder
from torchrec_b200.distributed.types import ParameterSharding, ShardingEnv, ShardingType
from torchrec_b200.modules.embedding_configs import PoolingType
from torchrec_b200.quant.embedding_modules import EmbeddingBagCollection as QuantEmbeddingBagCollection
from torchrec_b200.quant.embedding_modules import EmbeddingCollection as QuantEmbeddingCollection
from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor, KeyedTensor


def _device_for(rank: int, device_type: str) -> torch.device:
    return torch.device("cuda", rank) if device_type == "cuda" else torch.device(device_type)


class ShardedQuantEmbeddingBagCollection(nn.Module):
    def __init__(self, module: QuantEmbeddingBagCollection, table_name_to_parameter_sharding: Dict[str, ParameterSharding], env: ShardingEnv,
                 fused_params: Optional[Dict[str, Any]] = None, device: Optional[torch.device] = None) -> None:
        super().__init__()
        self._configs = module.embedding_bag_configs()
        self._is_weighted = module.is_weighted()
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
        self._names_per_rank: List[List[str]] = []
        for rank, cfgs in enumerate(by_rank):
            if not cfgs:
                self._shards.append(nn.Identity())
                self._feature_names_per_rank.append([])
                self._names_per_rank.append([])
                continue
            dev = _device_for(rank, self._device_type)
            shard = QuantEmbeddingBagCollection(copy.deepcopy(cfgs), self._is_weighted, dev, output_dtype=module.output_dtype())
            for cfg in cfgs:
                shard.embedding_bags[cfg.name].weight.copy_(module.embedding_bags[cfg.name].weight.to(dev))
            self._shards.append(shard)
            self._feature_names_per_rank.append([f for c in cfgs for f in c.feature_names])
        self._embedding_names = module._embedding_names
        self._length_per_key = module._length_per_key

    def forward(self, features: KeyedJaggedTensor) -> KeyedTensor:
        keys = features.keys()
        pieces: Dict[str, torch.Tensor] = {}
        for rank, (shard, fnames) in enumerate(zip(self._shards, self._feature_names_per_rank)):
            if not fnames:
                continue
            dev = _device_for(rank, self._device_type)
            local = features.permute([keys.index(f) for f in fnames]).to(dev, non_blocking=True)
            kt = shard(local)
            for k, v in kt.to_dict().items():
                pieces[k] = v.to(self._out_device, non_blocking=True)
        values = torch.cat([pieces[n] for n in self._embedding_names], dim=1)
        return KeyedTensor(keys=self._embedding_names, values=values, length_per_key=self._length_per_key)

    def sharded_parameter_names(self, prefix: str = ""):
        for rank, shard in enumerate(self._shards):
            if isinstance(shard, QuantEmbeddingBagCollection):
                for name in shard.embedding_bags.keys():
                    yield f"{prefix}_shards.{rank}.embedding_bags.{name}.weight"


class QuantEmbeddingBagCollectionSharder(BaseQuantEmbeddingSharder[QuantEmbeddingBagCollection]):
    def shard(self, module: QuantEmbeddingBagCollection, params: Dict[str, ParameterSharding], env: ShardingEnv,
              device: Optional[torch.device] = None, module_fqn: Optional[str] = None) -> ShardedQuantEmbeddingBagCollection:
        return ShardedQuantEmbeddingBagCollection(module, params, env, getattr(self, "fused_params", None), device)

    def shardable_parameters(self, module: QuantEmbeddingBagCollection) -> Dict[str, torch.Tensor]:
        return {name: m.weight for name, m in module.embedding_bags.items()}

    def sharding_types(self, compute_device_type: str) -> List[str]:
        return [ShardingType.TABLE_WISE.value]

    @property
    def module_type(self) -> Type[QuantEmbeddingBagCollection]:
        return QuantEmbeddingBagCollection
