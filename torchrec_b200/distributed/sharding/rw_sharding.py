"""Row-wise sharding: rows of every table are split in contiguous blocks over all ranks.

Input dist: bucketize each bag by owning row block (ids become shard-local), then a KJT all-to-all
with ``F`` keys per rank.  Lookup: SUM pooling even for MEAN tables (the divisor needs the whole
bag).  Output dist: reduce-scatter of the ``[W*B, D]`` partial sums.
Counterpart of ``torchrec/distributed/sharding/rw_sharding.py``.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Union

import torch
import torch.distributed as dist

from torchrec_b200.distributed.dist_data import (
    EmbeddingsAllToOneReduce,
    KJTAllToAll,
    PooledEmbeddingsReduceScatter,
    VariableBatchPooledEmbeddingsReduceScatter,
)
from torchrec_b200.distributed.embedding_lookup import GroupedPooledEmbeddingsLookup
from torchrec_b200.distributed.embedding_sharding import (
    BaseEmbeddingDist,
    BaseSparseFeaturesDist,
    EmbeddingShardingContext,
    EmbeddingShardingInfo,
    bucketize_kjt_before_all2all,
)
from torchrec_b200.distributed.embedding_types import BaseEmbeddingLookup, ShardedEmbeddingTable
from torchrec_b200.distributed.sharding.common import BaseSharding, C, F, T, W, global_metadata_of, make_sharded_table
from torchrec_b200.distributed.types import Awaitable, CommOp, NullShardingContext, QuantizedCommCodecs, ShardingEnv, ShardingType
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


def get_embedding_shard_metadata(grouped_embedding_configs_per_rank):
    """Shard metadata of every table of every rank, in rank-major order."""
    return [t.local_metadata for groups in grouped_embedding_configs_per_rank for g in groups for t in g.embedding_tables]


class BaseRwEmbeddingSharding(BaseSharding[C, F, T, W]):
    def __init__(self, sharding_infos: List[EmbeddingShardingInfo], env: ShardingEnv, device: Optional[torch.device] = None,
                 need_pos: bool = False, qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None) -> None:
        self._need_pos = need_pos
        super().__init__(sharding_infos, env, device if device is not None else torch.device("cpu"), qcomm_codecs_registry)
        self._has_feature_processor = any(g.has_feature_processor for g in self._grouped_embedding_configs)

    def _shard(self, sharding_infos: List[EmbeddingShardingInfo]) -> List[List[ShardedEmbeddingTable]]:
        tables_per_rank: List[List[ShardedEmbeddingTable]] = [[] for _ in range(self._world_size)]
        for info in sharding_infos:
            shards = info.param_sharding.sharding_spec.shards
            gm = global_metadata_of(info)
            for rank in range(self._world_size):
                tables_per_rank[rank].append(
                    make_sharded_table(info, shards[rank], gm, shards[rank].shard_sizes[0], info.embedding_config.embedding_dim)
                )
        return tables_per_rank

    # every rank holds a shard of every table: metadata is reported from this rank's groups
    def _flat(self, fn):
        return [x for g in self._grouped_embedding_configs for x in fn(g)]

    def embedding_shard_metadata(self):
        return [x for g in self._grouped_embedding_configs for x in g.embedding_shard_metadata()]

    def embedding_tables(self) -> List[ShardedEmbeddingTable]:
        return [t for g in self._grouped_embedding_configs for t in g.embedding_tables]

    def _get_num_features(self) -> int:
        return sum(g.num_features() for g in self._grouped_embedding_configs)

    def _get_feature_hash_sizes(self) -> List[int]:
        # in-training pruning routes by the unpruned id space (set by the sharded pruning collection before the first batch)
        override = getattr(self, "_table_hash_size_override", None)
        if override:
            return [override.get(t.name, t.num_embeddings) for g in self._grouped_embedding_configs for t in g.embedding_tables for _ in range(t.num_features())]
        return [h for g in self._grouped_embedding_configs for h in g.feature_hash_sizes()]

    def _get_feature_total_num_buckets(self) -> Optional[List[int]]:
        override = getattr(self, "_table_total_num_buckets_override", None)
        if override:
            return [override[t.name] for g in self._grouped_embedding_configs for t in g.embedding_tables for _ in range(t.num_features())]
        out: List[int] = []
        for g in self._grouped_embedding_configs:
            for t in g.embedding_tables:
                if t.total_num_buckets is not None:
                    out.extend([t.total_num_buckets] * t.num_features())
        return out if out else None


class RwSparseFeaturesDist(BaseSparseFeaturesDist[KeyedJaggedTensor]):
    """Bucketize by row block, then all-to-all with ``num_features`` keys per rank."""

    def __init__(self, pg: dist.ProcessGroup, num_features: int, feature_hash_sizes: List[int],
                 feature_total_num_buckets: Optional[List[int]] = None, device: Optional[torch.device] = None,
                 is_sequence: bool = False, has_feature_processor: bool = False, need_pos: bool = False,
                 keep_original_indices: bool = False) -> None:
        super().__init__()
        self._world_size: int = pg.size()
        self._num_features = num_features
        block_sizes = []
        for i, h in enumerate(feature_hash_sizes):
            div = self._world_size
            if feature_total_num_buckets is not None:
                assert feature_total_num_buckets[i] % self._world_size == 0
                div = feature_total_num_buckets[i]
            block_sizes.append((h + div - 1) // div)
        self.register_buffer("_feature_block_sizes_tensor", torch.tensor(block_sizes, device=device, dtype=torch.int64), persistent=False)
        self._has_multiple_blocks_per_shard = feature_total_num_buckets is not None
        if self._has_multiple_blocks_per_shard:
            self.register_buffer("_feature_total_num_blocks_tensor", torch.tensor(feature_total_num_buckets, device=device, dtype=torch.int64), persistent=False)
        self._dist = KJTAllToAll(pg=pg, splits=[self._num_features] * self._world_size)
        self._is_sequence = is_sequence
        self._has_feature_processor = has_feature_processor
        self._need_pos = need_pos
        self.unbucketize_permute_tensor: Optional[torch.Tensor] = None
        self._keep_original_indices = keep_original_indices

    def forward(self, sparse_features: KeyedJaggedTensor) -> Awaitable[Awaitable[KeyedJaggedTensor]]:
        bucketized, self.unbucketize_permute_tensor = bucketize_kjt_before_all2all(
            sparse_features,
            num_buckets=self._world_size,
            block_sizes=self._feature_block_sizes_tensor,
            total_num_blocks=self._feature_total_num_blocks_tensor if self._has_multiple_blocks_per_shard else None,
            output_permute=self._is_sequence,
            bucketize_pos=self._has_feature_processor if sparse_features.weights_or_none() is None else self._need_pos,
            keep_original_indices=self._keep_original_indices,
        )
        return self._dist(bucketized)


class RwPooledEmbeddingDist(BaseEmbeddingDist[EmbeddingShardingContext, torch.Tensor, torch.Tensor]):
    def __init__(self, pg: dist.ProcessGroup, embedding_dims: List[int], qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None) -> None:
        super().__init__()
        self._dist: Optional[Union[PooledEmbeddingsReduceScatter, VariableBatchPooledEmbeddingsReduceScatter]] = None
        self._pg = pg
        self._codecs = qcomm_codecs_registry.get(CommOp.POOLED_EMBEDDINGS_REDUCE_SCATTER.name, None) if qcomm_codecs_registry else None
        self._embedding_dims = embedding_dims

    def forward(self, local_embs: torch.Tensor, sharding_ctx: Optional[EmbeddingShardingContext] = None) -> Awaitable[torch.Tensor]:
        if self._dist is None:
            if sharding_ctx is not None and sharding_ctx.variable_batch_per_feature:
                self._dist = VariableBatchPooledEmbeddingsReduceScatter(pg=self._pg, codecs=self._codecs)
            else:
                self._dist = PooledEmbeddingsReduceScatter(pg=self._pg, codecs=self._codecs)
        if sharding_ctx is None:
            return self._dist(local_embs)
        if sharding_ctx.variable_batch_per_feature:
            return self._dist(local_embs, batch_size_per_rank_per_feature=sharding_ctx.batch_size_per_rank_per_feature, embedding_dims=self._embedding_dims)
        return self._dist(local_embs, input_splits=sharding_ctx.batch_size_per_rank or None)


class RwPooledEmbeddingSharding(BaseRwEmbeddingSharding[EmbeddingShardingContext, KeyedJaggedTensor, torch.Tensor, torch.Tensor]):
    sharding_type = ShardingType.ROW_WISE

    def create_input_dist(self, device: Optional[torch.device] = None) -> BaseSparseFeaturesDist[KeyedJaggedTensor]:
        return RwSparseFeaturesDist(
            pg=self._pg, num_features=self._get_num_features(), feature_hash_sizes=self._get_feature_hash_sizes(),
            feature_total_num_buckets=self._get_feature_total_num_buckets(), device=device if device is not None else self._device,
            is_sequence=False, has_feature_processor=self._has_feature_processor, need_pos=self._need_pos,
            keep_original_indices=getattr(self, "_keep_original_indices", False),
        )

    def create_lookup(self, device: Optional[torch.device] = None, fused_params: Optional[Dict[str, Any]] = None, feature_processor=None) -> BaseEmbeddingLookup:
        return GroupedPooledEmbeddingsLookup(
            grouped_configs=self._grouped_embedding_configs, pg=self._pg, device=device if device is not None else self._device,
            feature_processor=feature_processor, sharding_type=ShardingType.ROW_WISE,
        )

    def create_output_dist(self, device: Optional[torch.device] = None) -> BaseEmbeddingDist[EmbeddingShardingContext, torch.Tensor, torch.Tensor]:
        return RwPooledEmbeddingDist(self._pg, qcomm_codecs_registry=self.qcomm_codecs_registry, embedding_dims=self.embedding_dims())


class InferRwPooledEmbeddingDist(BaseEmbeddingDist[NullShardingContext, List[torch.Tensor], torch.Tensor]):
    def __init__(self, device: torch.device, world_size: int) -> None:
        super().__init__()
        self._dist = EmbeddingsAllToOneReduce(device=device, world_size=world_size)

    def forward(self, local_embs: List[torch.Tensor], sharding_ctx: Optional[NullShardingContext] = None) -> torch.Tensor:
        return self._dist(local_embs)


_INFER_NAMES = ("InferRwSparseFeaturesDist", "InferRwPooledEmbeddingSharding")


def __getattr__(name: str):
    """The inference strategies live in ``infer_shardings`` (they build on every training strategy); they are reachable from
    here under the reference's import path."""
    if name in _INFER_NAMES:
        from torchrec_b200.distributed.sharding import infer_shardings

        return getattr(infer_shardings, name)
    raise AttributeError(name)
