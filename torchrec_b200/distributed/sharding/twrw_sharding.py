"""Table-row-wise sharding: a table is assigned to one node and split by rows over that node's ranks.

Input dist: bucketize into ``local_size`` buckets, reorder keys so that each destination rank's
block is contiguous ("staggered shuffle"), KJT all-to-all with ``stagger = nodes``.  Output dist:
reduce-scatter inside the node, then an all-to-all across nodes.  On one NVSwitch box the node is
the world and the cross-node step is the identity.
Counterpart of ``torchrec/distributed/sharding/twrw_sharding.py``.
"""
from __future__ import annotations

import itertools
import math
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from torchrec_b200.distributed.comm import get_local_size, intra_and_cross_node_pg, intra_and_cross_node_pg_2D
from torchrec_b200.distributed.dist_data import KJTAllToAll, PooledEmbeddingsAllToAll, PooledEmbeddingsReduceScatter
from torchrec_b200.distributed.embedding_lookup import GroupedPooledEmbeddingsLookup
from torchrec_b200.distributed.embedding_sharding import (
    BaseEmbeddingDist,
    BaseSparseFeaturesDist,
    EmbeddingShardingContext,
    EmbeddingShardingInfo,
    bucketize_kjt_before_all2all,
)
from torchrec_b200.distributed.embedding_types import BaseEmbeddingLookup, GroupedEmbeddingConfig, ShardedEmbeddingTable
from torchrec_b200.distributed.sharding.common import BaseSharding, C, F, T, W, global_metadata_of, make_sharded_table
from torchrec_b200.distributed.types import Awaitable, CommOp, QuantizedCommCodecs, ShardingEnv, ShardingType
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class BaseTwRwEmbeddingSharding(BaseSharding[C, F, T, W]):
    def __init__(self, sharding_infos: List[EmbeddingShardingInfo], env: ShardingEnv, device: Optional[torch.device] = None,
                 need_pos: bool = False, qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None) -> None:
        self._need_pos = need_pos
        super().__init__(sharding_infos, env, device, qcomm_codecs_registry)
        self._grouped_embedding_configs_per_node: List[List[GroupedEmbeddingConfig]] = [
            self._grouped_embedding_configs_per_rank[rank] for rank in range(self._world_size) if rank % self._local_size == 0
        ]
        self._has_feature_processor = any(g.has_feature_processor for g in self._grouped_embedding_configs_per_rank[self._rank])

    def _post_env_init(self) -> None:
        if self._is_2D_parallel:
            intra_pg, cross_pg = intra_and_cross_node_pg_2D(self._env, device=self._device)
        elif self._pg is not None:
            intra_pg, cross_pg = intra_and_cross_node_pg(self._device, backend=dist.get_backend(self._pg))
        else:
            intra_pg, cross_pg = None, None
        self._intra_pg, self._cross_pg = intra_pg, cross_pg
        self._local_size: int = intra_pg.size() if intra_pg else get_local_size(self._world_size)

    def _shard(self, sharding_infos: List[EmbeddingShardingInfo]) -> List[List[ShardedEmbeddingTable]]:
        tables_per_rank: List[List[ShardedEmbeddingTable]] = [[] for _ in range(self._world_size)]
        L = self._local_size
        for info in sharding_infos:
            node = info.param_sharding.ranks[0] // L
            shards = info.param_sharding.sharding_spec.shards
            gm = global_metadata_of(info)
            for rank in range(node * L, (node + 1) * L):
                i = rank - node * L
                tables_per_rank[rank].append(make_sharded_table(info, shards[i], gm, shards[i].shard_sizes[0], info.embedding_config.embedding_dim))
        return tables_per_rank

    def _per_node(self, fn) -> List[Any]:
        return [x for groups in self._grouped_embedding_configs_per_node for g in groups for x in fn(g)]

    def embedding_dims(self) -> List[int]:
        return self._per_node(lambda g: g.embedding_dims())

    def embedding_names(self) -> List[str]:
        return self._per_node(lambda g: g.embedding_names())

    def embedding_shard_metadata(self):
        return self._per_node(lambda g: g.embedding_shard_metadata())

    def feature_names(self) -> List[str]:
        return self._per_node(lambda g: g.feature_names())

    def embedding_tables(self) -> List[ShardedEmbeddingTable]:
        return self._per_node(lambda g: g.embedding_tables)

    def _get_feature_hash_sizes(self) -> List[int]:
        return self._per_node(lambda g: g.feature_hash_sizes())

    def _dim_sum_per_node(self) -> List[int]:
        return [sum(g.dim_sum() for g in groups) for groups in self._grouped_embedding_configs_per_node]

    def _emb_dim_per_node_per_feature(self) -> List[List[int]]:
        return [[d for g in groups for d in g.embedding_dims()] for groups in self._grouped_embedding_configs_per_node]

    def _features_per_rank(self, group: List[List[GroupedEmbeddingConfig]]) -> List[int]:
        return [sum(g.num_features() for g in groups) for groups in group]


class TwRwSparseFeaturesDist(BaseSparseFeaturesDist[KeyedJaggedTensor]):
    def __init__(self, pg: dist.ProcessGroup, local_size: int, features_per_rank: List[int], feature_hash_sizes: List[int],
                 device: Optional[torch.device] = None, has_feature_processor: bool = False, need_pos: bool = False) -> None:
        super().__init__()
        assert pg.size() % local_size == 0, "currently group granularity must be node"
        self._world_size = pg.size()
        self._local_size = local_size
        self._num_cross_nodes = self._world_size // self._local_size
        block_sizes = [math.ceil(h / self._local_size) for h in feature_hash_sizes]
        self._sf_staggered_shuffle = self._staggered_shuffle(features_per_rank)
        self.register_buffer("_feature_block_sizes_tensor", torch.tensor(block_sizes, device=device, dtype=torch.int64), persistent=False)
        self.register_buffer("_sf_staggered_shuffle_tensor", torch.tensor(self._sf_staggered_shuffle, device=device, dtype=torch.int32), persistent=False)
        self._dist = KJTAllToAll(pg=pg, splits=features_per_rank, stagger=self._num_cross_nodes)
        self._has_feature_processor = has_feature_processor
        self._need_pos = need_pos

    def forward(self, sparse_features: KeyedJaggedTensor) -> Awaitable[Awaitable[KeyedJaggedTensor]]:
        bucketized = bucketize_kjt_before_all2all(
            sparse_features, num_buckets=self._local_size, block_sizes=self._feature_block_sizes_tensor, output_permute=False,
            bucketize_pos=self._has_feature_processor if sparse_features.weights_or_none() is None else self._need_pos,
        )[0].permute(self._sf_staggered_shuffle, self._sf_staggered_shuffle_tensor)
        return self._dist(bucketized)

    def _staggered_shuffle(self, features_per_rank: List[int]) -> List[int]:
        nodes = self._world_size // self._local_size
        features_per_node = [features_per_rank[node * self._local_size] for node in range(nodes)]
        node_offsets = [0] + list(itertools.accumulate(features_per_node))
        num_features = node_offsets[-1]
        return [
            bucket * num_features + feature
            for node in range(nodes) for bucket in range(self._local_size)
            for feature in range(node_offsets[node], node_offsets[node + 1])
        ]


class TwRwPooledEmbeddingDist(BaseEmbeddingDist[EmbeddingShardingContext, torch.Tensor, torch.Tensor]):
    """Reduce-scatter inside the node, wait, then all-to-all across nodes."""

    def __init__(self, rank: int, cross_pg: dist.ProcessGroup, intra_pg: dist.ProcessGroup, dim_sum_per_node: List[int],
                 emb_dim_per_node_per_feature: List[List[int]], device: Optional[torch.device] = None,
                 qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None,
                 callbacks=None) -> None:
        super().__init__()
        self._rank = rank
        self._intra_pg, self._cross_pg = intra_pg, cross_pg
        intra_codecs = qcomm_codecs_registry.get(CommOp.POOLED_EMBEDDINGS_REDUCE_SCATTER.name, None) if qcomm_codecs_registry else None
        cross_codecs = qcomm_codecs_registry.get(CommOp.POOLED_EMBEDDINGS_ALL_TO_ALL.name, None) if qcomm_codecs_registry else None
        self._intra_dist = PooledEmbeddingsReduceScatter(intra_pg, codecs=intra_codecs)
        self._cross_dist = PooledEmbeddingsAllToAll(cross_pg, dim_sum_per_node, device, callbacks=callbacks, codecs=cross_codecs)

    def forward(self, local_embs: torch.Tensor, sharding_ctx: Optional[EmbeddingShardingContext] = None) -> Awaitable[torch.Tensor]:
        if sharding_ctx is not None and sharding_ctx.variable_batch_per_feature:
            raise NotImplementedError("variable batch per feature is not supported with table-row-wise sharding")
        if sharding_ctx is not None and len(set(sharding_ctx.batch_size_per_rank)) > 1:
            per_cross, sums = self._preprocess_batch_size_per_rank(self._intra_pg.size(), self._cross_pg.size(), sharding_ctx.batch_size_per_rank)
            rs = self._intra_dist(local_embs, input_splits=sums).wait()
            return self._cross_dist(rs, batch_size_per_rank=per_cross[self._rank % self._intra_pg.size()])
        return self._cross_dist(self._intra_dist(local_embs).wait())

    @staticmethod
    def _preprocess_batch_size_per_rank(local_size: int, nodes: int, batch_size_per_rank: List[int]) -> Tuple[List[List[int]], List[int]]:
        per_cross, sums = [], []
        for lr in range(local_size):
            bs = [batch_size_per_rank[lr + node * local_size] for node in range(nodes)]
            per_cross.append(bs)
            sums.append(sum(bs))
        return per_cross, sums


class TwRwPooledEmbeddingSharding(BaseTwRwEmbeddingSharding[EmbeddingShardingContext, KeyedJaggedTensor, torch.Tensor, torch.Tensor]):
    sharding_type = ShardingType.TABLE_ROW_WISE

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
        return TwRwPooledEmbeddingDist(
            rank=self._rank, cross_pg=self._cross_pg, intra_pg=self._intra_pg, dim_sum_per_node=self._dim_sum_per_node(),
            emb_dim_per_node_per_feature=self._emb_dim_per_node_per_feature(), device=device if device is not None else self._device,
            qcomm_codecs_registry=self.qcomm_codecs_registry,
        )
