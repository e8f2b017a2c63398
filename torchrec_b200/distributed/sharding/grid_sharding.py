"""Grid sharding: column shards, each placed on a node and split by rows over that node's ranks
(column-wise across nodes x table-row-wise inside a node).
Counterpart of ``torchrec/distributed/sharding/grid_sharding.py``.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Set, Tuple

import torch

from torchrec_b200.distributed.embedding_lookup import GroupedPooledEmbeddingsLookup
from torchrec_b200.distributed.embedding_sharding import BaseEmbeddingDist, BaseSparseFeaturesDist, EmbeddingShardingContext, EmbeddingShardingInfo
from torchrec_b200.distributed.embedding_types import BaseEmbeddingLookup, ShardedEmbeddingTable
from torchrec_b200.distributed.sharding.common import C, F, T, W, global_metadata_of, make_sharded_table
from torchrec_b200.distributed.sharding.cw_sharding import PermutePooledEmbeddingsSplit
from torchrec_b200.distributed.sharding.twrw_sharding import BaseTwRwEmbeddingSharding, TwRwPooledEmbeddingDist, TwRwSparseFeaturesDist
from torchrec_b200.distributed.types import QuantizedCommCodecs, ShardingEnv, ShardingType
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class BaseGridEmbeddingSharding(BaseTwRwEmbeddingSharding[C, F, T, W]):
    def __init__(self, sharding_infos: List[EmbeddingShardingInfo], env: ShardingEnv, device: Optional[torch.device] = None,
                 need_pos: bool = False, qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None) -> None:
        super().__init__(sharding_infos, env, device, need_pos, qcomm_codecs_registry)
        self._init_combined_embeddings()

    def _shard(self, sharding_infos: List[EmbeddingShardingInfo]) -> List[List[ShardedEmbeddingTable]]:
        tables_per_rank: List[List[ShardedEmbeddingTable]] = [[] for _ in range(self._world_size)]
        for info in sharding_infos:
            shards = info.param_sharding.sharding_spec.shards
            gm = global_metadata_of(info)
            for i, rank in enumerate(info.param_sharding.ranks):
                tables_per_rank[rank].append(make_sharded_table(info, shards[i], gm, shards[i].shard_sizes[0], shards[i].shard_sizes[1]))
        return tables_per_rank

    def _init_combined_embeddings(self) -> None:
        names = super().embedding_names()
        dims = super().embedding_dims()
        metas = super().embedding_shard_metadata()
        by_name: Dict[str, List[Tuple[int, int]]] = {}
        for i, (n, md) in enumerate(zip(names, metas)):
            by_name.setdefault(n, []).append((i, md.shard_offsets[1] if md is not None else 0))
        name_to_index = {n: [i for i, _ in sorted(v, key=lambda t: t[1])] for n, v in by_name.items()}
        combined_names, seen = [], set()
        for n in names:
            if n not in seen:
                combined_names.append(n)
                seen.add(n)
        combined_dims, order = [], []
        for n in combined_names:
            combined_dims.append(sum(dims[i] for i in name_to_index[n]))
            order.extend(name_to_index[n])
        self._embedding_names, self._embedding_dims, self._embedding_order = names, dims, order
        self._combined_embedding_names, self._combined_embedding_dims = combined_names, combined_dims

    def embedding_dims(self) -> List[int]:
        return self._combined_embedding_dims

    def embedding_names(self) -> List[str]:
        return self._combined_embedding_names

    def uncombined_embedding_dims(self) -> List[int]:
        return self._embedding_dims

    def uncombined_embedding_names(self) -> List[str]:
        return self._embedding_names


class GridPooledEmbeddingSharding(BaseGridEmbeddingSharding[EmbeddingShardingContext, KeyedJaggedTensor, torch.Tensor, torch.Tensor]):
    sharding_type = ShardingType.GRID_SHARD

    def create_input_dist(self, device: Optional[torch.device] = None) -> BaseSparseFeaturesDist[KeyedJaggedTensor]:
        return TwRwSparseFeaturesDist(
            pg=self._pg, local_size=self._local_size, features_per_rank=self._features_per_rank(self._grouped_embedding_configs_per_rank),
            feature_hash_sizes=self._get_feature_hash_sizes(), device=device if device is not None else self._device,
            has_feature_processor=self._has_feature_processor, need_pos=self._need_pos,
        )

    def create_lookup(self, device: Optional[torch.device] = None, fused_params: Optional[Dict[str, Any]] = None, feature_processor=None) -> BaseEmbeddingLookup:
        return GroupedPooledEmbeddingsLookup(
            grouped_configs=self._grouped_embedding_configs_per_rank[self._rank], pg=self._pg,
            device=device if device is not None else self._device, feature_processor=feature_processor,
            sharding_type=ShardingType.TABLE_ROW_WISE,
        )

    def create_output_dist(self, device: Optional[torch.device] = None) -> BaseEmbeddingDist[EmbeddingShardingContext, torch.Tensor, torch.Tensor]:
        callbacks = None
        if self._embedding_order != list(range(len(self._embedding_order))):
            callbacks = [PermutePooledEmbeddingsSplit(self._embedding_dims, self._embedding_order, device=device)]
        return TwRwPooledEmbeddingDist(
            rank=self._rank, cross_pg=self._cross_pg, intra_pg=self._intra_pg, dim_sum_per_node=self._dim_sum_per_node(),
            emb_dim_per_node_per_feature=self._emb_dim_per_node_per_feature(), device=device if device is not None else self._device,
            qcomm_codecs_registry=self.qcomm_codecs_registry, callbacks=callbacks,
        )
