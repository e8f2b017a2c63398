"""Table-wise sharding: every table lives entirely on one rank.

Input dist: key-split KJT all-to-all (rank r receives the features of its tables for the global
batch).  Output dist: pooled all-to-all ``[B_global, D_local] -> [B_local, sum D]``.
Counterpart of ``torchrec/distributed/sharding/tw_sharding.py``.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional, TypeVar

import torch
import torch.distributed as dist

from torchrec_b200.distributed.dist_data import (
    EmbeddingsAllToOne,
    KJTAllToAll,
    KJTOneToAll,
    PooledEmbeddingsAllToAll,
    VariableBatchPooledEmbeddingsAllToAll,
)
from torchrec_b200.distributed.embedding_lookup import GroupedPooledEmbeddingsLookup
from torchrec_b200.distributed.embedding_sharding import (
    BaseEmbeddingDist,
    BaseSparseFeaturesDist,
    EmbeddingShardingContext,
    EmbeddingShardingInfo,
)
from torchrec_b200.distributed.embedding_types import BaseEmbeddingLookup, InputDistOutputs, KJTList, ShardedEmbeddingTable
from torchrec_b200.distributed.sharding.common import BaseSharding, C, F, T, W, global_metadata_of, make_sharded_table
from torchrec_b200.distributed.types import Awaitable, CommOp, NoWait, NullShardingContext, QuantizedCommCodecs, ShardingType
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class BaseTwEmbeddingSharding(BaseSharding[C, F, T, W]):
    def _shard(self, sharding_infos: List[EmbeddingShardingInfo]) -> List[List[ShardedEmbeddingTable]]:
        tables_per_rank: List[List[ShardedEmbeddingTable]] = [[] for _ in range(self._world_size)]
        for info in sharding_infos:
            shards = info.param_sharding.sharding_spec.shards
            cfg = info.embedding_config
            rows = cfg.num_embeddings_post_pruning if cfg.num_embeddings_post_pruning is not None else cfg.num_embeddings
            rank = self._remap(info.param_sharding.ranks[0], ShardingType.TABLE_WISE)
            tables_per_rank[rank].append(make_sharded_table(info, shards[0], global_metadata_of(info), rows, cfg.embedding_dim))
        return tables_per_rank


class TwSparseFeaturesDist(BaseSparseFeaturesDist[KeyedJaggedTensor]):
    def __init__(self, pg: dist.ProcessGroup, features_per_rank: List[int]) -> None:
        super().__init__()
        self._dist = KJTAllToAll(pg=pg, splits=features_per_rank)

    def forward(self, sparse_features: KeyedJaggedTensor) -> Awaitable[Awaitable[KeyedJaggedTensor]]:
        return self._dist(sparse_features)


class TwPooledEmbeddingDist(BaseEmbeddingDist[EmbeddingShardingContext, torch.Tensor, torch.Tensor]):
    def __init__(self, pg: dist.ProcessGroup, dim_sum_per_rank: List[int], emb_dim_per_rank_per_feature: List[List[int]],
                 device: Optional[torch.device] = None, callbacks: Optional[List[Callable[[torch.Tensor], torch.Tensor]]] = None,
                 qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None) -> None:
        super().__init__()
        self._pg = pg
        self._dim_sum_per_rank = dim_sum_per_rank
        self._device = device
        self._callbacks = callbacks
        self._codecs = qcomm_codecs_registry.get(CommOp.POOLED_EMBEDDINGS_ALL_TO_ALL.name, None) if qcomm_codecs_registry else None
        self._emb_dim_per_rank_per_feature = emb_dim_per_rank_per_feature
        self._dist: Optional[PooledEmbeddingsAllToAll] = None
        self._variable_dist: Optional[VariableBatchPooledEmbeddingsAllToAll] = None

    def forward(self, local_embs: torch.Tensor, sharding_ctx: Optional[EmbeddingShardingContext] = None) -> Awaitable[torch.Tensor]:
        if self._dist is None:
            self._create_output_dist_module(sharding_ctx)
        if sharding_ctx is None:
            return self._dist(local_embs)
        if sharding_ctx.variable_batch_per_feature:
            return self._variable_dist(
                local_embs, batch_size_per_rank_per_feature=sharding_ctx.batch_size_per_rank_per_feature,
                batch_size_per_feature_pre_a2a=sharding_ctx.batch_size_per_feature_pre_a2a,
            )
        return self._dist(local_embs, batch_size_per_rank=sharding_ctx.batch_size_per_rank or None)

    def _create_output_dist_module(self, sharding_ctx: Optional[EmbeddingShardingContext] = None) -> None:
        if sharding_ctx is not None and sharding_ctx.variable_batch_per_feature:
            self._variable_dist = VariableBatchPooledEmbeddingsAllToAll(
                pg=self._pg, emb_dim_per_rank_per_feature=self._emb_dim_per_rank_per_feature, device=self._device, codecs=self._codecs,
            )
        self._dist = PooledEmbeddingsAllToAll(
            pg=self._pg, dim_sum_per_rank=self._dim_sum_per_rank, device=self._device, callbacks=self._callbacks, codecs=self._codecs,
        )


class TwPooledEmbeddingSharding(BaseTwEmbeddingSharding[EmbeddingShardingContext, KeyedJaggedTensor, torch.Tensor, torch.Tensor]):
    sharding_type = ShardingType.TABLE_WISE

    def create_input_dist(self, device: Optional[torch.device] = None) -> BaseSparseFeaturesDist[KeyedJaggedTensor]:
        assert self._pg is not None
        return TwSparseFeaturesDist(self._pg, self.features_per_rank())

    def create_lookup(self, device: Optional[torch.device] = None, fused_params: Optional[Dict[str, Any]] = None, feature_processor=None) -> BaseEmbeddingLookup:
        lookup = GroupedPooledEmbeddingsLookup(
            grouped_configs=self._grouped_embedding_configs, pg=self._pg, device=device if device is not None else self._device,
            feature_processor=feature_processor, sharding_type=ShardingType.TABLE_WISE,
        )
        return lookup

    def create_output_dist(self, device: Optional[torch.device] = None) -> BaseEmbeddingDist[EmbeddingShardingContext, torch.Tensor, torch.Tensor]:
        assert self._pg is not None
        return TwPooledEmbeddingDist(
            pg=self._pg, dim_sum_per_rank=self._dim_sum_per_rank(), emb_dim_per_rank_per_feature=self._emb_dim_per_rank_per_feature(),
            device=device if device is not None else self._device, qcomm_codecs_registry=self.qcomm_codecs_registry,
        )


# ---- inference (one process, all devices) ------------------------------------------------------------
class InferTwSparseFeaturesDist(BaseSparseFeaturesDist[InputDistOutputs]):
    def __init__(self, features_per_rank: List[int], world_size: int, device: Optional[torch.device] = None) -> None:
        super().__init__()
        self._dist = KJTOneToAll(splits=features_per_rank, world_size=world_size, device=device)

    def forward(self, sparse_features: KeyedJaggedTensor) -> InputDistOutputs:
        return InputDistOutputs(features=self._dist.forward(sparse_features).wait())


class InferTwPooledEmbeddingDist(BaseEmbeddingDist[NullShardingContext, List[torch.Tensor], torch.Tensor]):
    def __init__(self, device: torch.device, world_size: int) -> None:
        super().__init__()
        self._dist = EmbeddingsAllToOne(device, world_size, 1)

    def forward(self, local_embs: List[torch.Tensor], sharding_ctx: Optional[NullShardingContext] = None) -> torch.Tensor:
        return self._dist(local_embs)
