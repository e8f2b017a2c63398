"""Data-parallel "sharding": every rank holds the full table and looks up its own batch; the dense
weight gradient is all-reduced by DDP.  Counterpart of ``torchrec/distributed/sharding/dp_sharding.py``.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch

from torchrec_b200.distributed.embedding_lookup import GroupedPooledEmbeddingsLookup
from torchrec_b200.distributed.embedding_sharding import (
    BaseEmbeddingDist,
    BaseSparseFeaturesDist,
    EmbeddingShardingContext,
    EmbeddingShardingInfo,
)
from torchrec_b200.distributed.embedding_types import BaseEmbeddingLookup, ShardedEmbeddingTable
from torchrec_b200.distributed.sharding.common import BaseSharding, C, F, T, W, make_sharded_table
from torchrec_b200.distributed.types import Awaitable, NoWait, ShardingType
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class BaseDpEmbeddingSharding(BaseSharding[C, F, T, W]):
    def _shard(self, sharding_infos: List[EmbeddingShardingInfo]) -> List[List[ShardedEmbeddingTable]]:
        tables_per_rank: List[List[ShardedEmbeddingTable]] = [[] for _ in range(self._world_size)]
        for info in sharding_infos:
            cfg = info.embedding_config
            for rank in range(self._world_size):
                tables_per_rank[rank].append(make_sharded_table(info, None, None, cfg.num_embeddings, cfg.embedding_dim))
        return tables_per_rank

    # every rank has the same tables: report rank 0's view once
    def _flat(self, fn):
        return [x for g in self._grouped_embedding_configs for x in fn(g)]

    def embedding_names_per_rank(self) -> List[List[str]]:
        raise NotImplementedError

    def feature_names_per_rank(self) -> List[List[str]]:
        raise NotImplementedError

    def embedding_tables(self) -> List[ShardedEmbeddingTable]:
        return [t for g in self._grouped_embedding_configs for t in g.embedding_tables]


class DpSparseFeaturesDist(BaseSparseFeaturesDist[KeyedJaggedTensor]):
    def forward(self, sparse_features: KeyedJaggedTensor) -> Awaitable[Awaitable[KeyedJaggedTensor]]:
        return NoWait(NoWait(sparse_features))


class DpPooledEmbeddingDist(BaseEmbeddingDist[EmbeddingShardingContext, torch.Tensor, torch.Tensor]):
    def forward(self, local_embs: torch.Tensor, sharding_ctx: Optional[EmbeddingShardingContext] = None) -> Awaitable[torch.Tensor]:
        return NoWait(local_embs)


class DpPooledEmbeddingSharding(BaseDpEmbeddingSharding[EmbeddingShardingContext, KeyedJaggedTensor, torch.Tensor, torch.Tensor]):
    sharding_type = ShardingType.DATA_PARALLEL

    def create_input_dist(self, device: Optional[torch.device] = None) -> BaseSparseFeaturesDist[KeyedJaggedTensor]:
        return DpSparseFeaturesDist()

    def create_lookup(self, device: Optional[torch.device] = None, fused_params: Optional[Dict[str, Any]] = None, feature_processor=None) -> BaseEmbeddingLookup:
        return GroupedPooledEmbeddingsLookup(
            grouped_configs=self._grouped_embedding_configs, pg=self._env.process_group,
            device=device if device is not None else self._device, feature_processor=feature_processor,
            scale_weight_gradients=False, sharding_type=ShardingType.DATA_PARALLEL,
        )

    def create_output_dist(self, device: Optional[torch.device] = None) -> BaseEmbeddingDist[EmbeddingShardingContext, torch.Tensor, torch.Tensor]:
        return DpPooledEmbeddingDist()
