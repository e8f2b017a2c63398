"""Adapters that give a plain embedding-collection interface to a managed-collision collection: construct from the same table
configs, call with a KJT, get the collection's usual output; the remapped ids of the last call are kept on the adapter.
``zch_method`` picks the remapper of every table: ``"mpzch"`` (bucketed hash probing with TTL eviction) or ``"sort_zch"``
(sorted table with distance-LFU eviction).  Counterpart of ``torchrec/modules/mc_adapter.py:36-260``."""
from __future__ import annotations

from typing import Dict, Iterator, List, Optional, Sequence

import torch
from torch import nn
from torch.nn.parameter import Parameter

from torchrec_b200.modules.embedding_configs import BaseEmbeddingConfig, EmbeddingBagConfig, EmbeddingConfig
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection, EmbeddingCollection
from torchrec_b200.modules.hash_mc_evictions import HashZchEvictionConfig, HashZchEvictionPolicyName
from torchrec_b200.modules.hash_mc_modules import HashZchManagedCollisionModule
from torchrec_b200.modules.mc_embedding_modules import ManagedCollisionEmbeddingBagCollection, ManagedCollisionEmbeddingCollection
from torchrec_b200.modules.mc_modules import DistanceLFU_EvictionPolicy, ManagedCollisionCollection, ManagedCollisionModule, MCHManagedCollisionModule
from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor, KeyedTensor


def _remappers_for(configs: Sequence[BaseEmbeddingConfig], zch_method: str, input_hash_size: int, device: torch.device, world_size: int,
                   eviction_interval: int, mpzch_num_buckets: Optional[int], mpzch_max_probe: Optional[int]) -> Dict[str, ManagedCollisionModule]:
    out: Dict[str, ManagedCollisionModule] = {}
    for cfg in configs:
        if zch_method == "mpzch":
            out[cfg.name] = HashZchManagedCollisionModule(
                zch_size=cfg.num_embeddings, device=device, total_num_buckets=mpzch_num_buckets or world_size,
                max_probe=mpzch_max_probe or 128, input_hash_size=input_hash_size, is_inference=False,
                eviction_policy_name=HashZchEvictionPolicyName.SINGLE_TTL_EVICTION,
                eviction_config=HashZchEvictionConfig(features=list(cfg.feature_names), single_ttl=eviction_interval))
        elif zch_method == "sort_zch":
            out[cfg.name] = MCHManagedCollisionModule(zch_size=cfg.num_embeddings, device=device, input_hash_size=input_hash_size,
                                                      eviction_interval=eviction_interval, eviction_policy=DistanceLFU_EvictionPolicy())
        else:
            raise NotImplementedError(f"zc method {zch_method!r} is not supported; use 'mpzch' or 'sort_zch'")
    return out


class McEmbeddingCollectionAdapter(nn.Module):
    """``forward(KJT) -> Dict[feature, JaggedTensor]`` through id remapping.  ``parameters()`` yields the embedding weights only."""

    def __init__(self, tables: List[EmbeddingConfig], input_hash_size: int, device: torch.device, world_size: int, eviction_interval: int = 1,
                 allow_in_place_embed_weight_update: bool = False, zch_method: str = "", mpzch_num_buckets: Optional[int] = 80,
                 mpzch_max_probe: Optional[int] = 100) -> None:
        super().__init__()
        ec = EmbeddingCollection(tables=tables, device=torch.device("meta"))
        remappers = _remappers_for(ec.embedding_configs(), zch_method, input_hash_size, device, world_size, eviction_interval, mpzch_num_buckets, mpzch_max_probe)
        self.mc_embedding_collection = ManagedCollisionEmbeddingCollection(
            ec, ManagedCollisionCollection(managed_collision_modules=remappers, embedding_configs=ec.embedding_configs()), return_remapped_features=False)
        self.allow_in_place_embed_weight_update = allow_in_place_embed_weight_update
        self.remapped_ids: Optional[KeyedJaggedTensor] = None

    def forward(self, input: KeyedJaggedTensor) -> Dict[str, JaggedTensor]:
        out, self.remapped_ids = self.mc_embedding_collection(input)
        return out

    def parameters(self, recurse: bool = True) -> Iterator[Parameter]:
        return self.mc_embedding_collection._embedding_module.parameters(recurse=recurse)

    def embedding_bag_configs(self) -> List[EmbeddingConfig]:
        return self.mc_embedding_collection._embedding_module.embedding_configs()


class McEmbeddingBagCollectionAdapter(nn.Module):
    """``forward(KJT) -> KeyedTensor`` through id remapping.  ``parameters()`` yields the embedding weights only."""

    def __init__(self, tables: List[EmbeddingBagConfig], input_hash_size: int, device: torch.device, world_size: int, eviction_interval: int = 1,
                 allow_in_place_embed_weight_update: bool = False, zch_method: str = "", mpzch_num_buckets: Optional[int] = 80,
                 mpzch_max_probe: Optional[int] = 100) -> None:
        super().__init__()
        ebc = EmbeddingBagCollection(tables=tables, device=torch.device("meta"))
        remappers = _remappers_for(ebc.embedding_bag_configs(), zch_method, input_hash_size, device, world_size, eviction_interval, mpzch_num_buckets, mpzch_max_probe)
        self.mc_embedding_bag_collection = ManagedCollisionEmbeddingBagCollection(
            ebc, ManagedCollisionCollection(managed_collision_modules=remappers, embedding_configs=ebc.embedding_bag_configs()), return_remapped_features=False)
        self.allow_in_place_embed_weight_update = allow_in_place_embed_weight_update
        self.remapped_ids: Optional[KeyedJaggedTensor] = None

    def forward(self, input: KeyedJaggedTensor) -> KeyedTensor:
        out, self.remapped_ids = self.mc_embedding_bag_collection(input)
        return out

    def parameters(self, recurse: bool = True) -> Iterator[Parameter]:
        return self.mc_embedding_bag_collection._embedding_module.parameters(recurse=recurse)

    def embedding_bag_configs(self) -> List[EmbeddingBagConfig]:
        return self.mc_embedding_bag_collection._embedding_module.embedding_bag_configs()
