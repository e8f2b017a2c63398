"""Logic shared by every sharding strategy: shard bookkeeping and the accessor surface.

The reference repeats these accessors in each ``sharding/*_sharding.py`` (e.g.
``torchrec/distributed/sharding/tw_sharding.py:189-268``); here they live once.
"""
from __future__ import annotations

from typing import Any, Dict, Generic, List, Optional, TypeVar

import torch
import torch.distributed as dist

from torchrec_b200.distributed.embedding_sharding import (
    EmbeddingSharding,
    EmbeddingShardingInfo,
    group_tables,
)
from torchrec_b200.distributed.embedding_types import (
    EmbeddingComputeKernel,
    GroupedEmbeddingConfig,
    ShardedEmbeddingTable,
)
from torchrec_b200.distributed.types import (
    QuantizedCommCodecs,
    ShardedTensorMetadata,
    ShardingEnv,
    ShardingEnv2D,
    ShardMetadata,
)
from torchrec_b200.streamable import Multistreamable

C = TypeVar("C", bound=Multistreamable)
F = TypeVar("F", bound=Multistreamable)
T = TypeVar("T")
W = TypeVar("W")


def make_sharded_table(info: EmbeddingShardingInfo, local_metadata: Optional[ShardMetadata], global_metadata: Optional[ShardedTensorMetadata],
                       local_rows: int, local_cols: int, dtensor_metadata: Any = None) -> ShardedEmbeddingTable:
    cfg = info.embedding_config
    return ShardedEmbeddingTable(
        num_embeddings=cfg.num_embeddings,
        embedding_dim=cfg.embedding_dim,
        name=cfg.name,
        embedding_names=cfg.embedding_names,
        data_type=cfg.data_type,
        feature_names=cfg.feature_names,
        pooling=cfg.pooling,
        is_weighted=cfg.is_weighted,
        has_feature_processor=cfg.has_feature_processor,
        local_rows=local_rows,
        local_cols=local_cols,
        compute_kernel=EmbeddingComputeKernel(info.param_sharding.compute_kernel),
        local_metadata=local_metadata,
        global_metadata=global_metadata,
        dtensor_metadata=dtensor_metadata,
        weight_init_max=cfg.weight_init_max,
        weight_init_min=cfg.weight_init_min,
        init_fn=cfg.init_fn,
        fused_params=info.fused_params,
        num_embeddings_post_pruning=cfg.num_embeddings_post_pruning,
        use_virtual_table=cfg.use_virtual_table,
        need_pos=cfg.need_pos,
        total_num_buckets=cfg.total_num_buckets,
    )


def global_metadata_of(info: EmbeddingShardingInfo) -> ShardedTensorMetadata:
    cfg = info.embedding_config
    rows = cfg.num_embeddings_post_pruning if cfg.num_embeddings_post_pruning is not None else cfg.num_embeddings
    return ShardedTensorMetadata(shards_metadata=info.param_sharding.sharding_spec.shards, size=torch.Size([rows, cfg.embedding_dim]))


class BaseSharding(EmbeddingSharding[C, F, T, W]):
    """Holds ``tables_per_rank`` -> TBE groups per rank and answers every metadata query."""

    def __init__(self, sharding_infos: List[EmbeddingShardingInfo], env: ShardingEnv, device: Optional[torch.device] = None,
                 qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None) -> None:
        super().__init__(qcomm_codecs_registry=qcomm_codecs_registry)
        self._env = env
        self._device = device
        self._is_2D_parallel = isinstance(env, ShardingEnv2D)
        self._pg: Optional[dist.ProcessGroup] = env.sharding_pg if self._is_2D_parallel else env.process_group  # type: ignore[attr-defined]
        self._world_size: int = env.world_size
        self._rank: int = env.rank
        self._sharding_infos = sharding_infos
        self._post_env_init()
        self._sharded_tables_per_rank: List[List[ShardedEmbeddingTable]] = self._shard(sharding_infos)
        self._grouped_embedding_configs_per_rank: List[List[GroupedEmbeddingConfig]] = group_tables(self._sharded_tables_per_rank)
        self._grouped_embedding_configs: List[GroupedEmbeddingConfig] = self._grouped_embedding_configs_per_rank[self._rank]

    def _post_env_init(self) -> None:
        """Hook for subclasses that need topology (node size, sub-groups) before ``_shard`` runs."""

    def _shard(self, sharding_infos: List[EmbeddingShardingInfo]) -> List[List[ShardedEmbeddingTable]]:
        raise NotImplementedError

    def _remap(self, rank: int, sharding_type) -> int:
        return self._env.remap_rank(rank, sharding_type) if self._is_2D_parallel else rank  # type: ignore[attr-defined]

    def _per_rank(self, fn) -> List[Any]:
        return [[x for g in groups for x in fn(g)] for groups in self._grouped_embedding_configs_per_rank]

    def _flat(self, fn) -> List[Any]:
        return [x for groups in self._grouped_embedding_configs_per_rank for g in groups for x in fn(g)]

    def _dim_sum_per_rank(self) -> List[int]:
        return [sum(g.dim_sum() for g in groups) for groups in self._grouped_embedding_configs_per_rank]

    def _emb_dim_per_rank_per_feature(self) -> List[List[int]]:
        return self._per_rank(lambda g: g.embedding_dims())

    def embedding_dims(self) -> List[int]:
        return self._flat(lambda g: g.embedding_dims())

    def embedding_names(self) -> List[str]:
        return self._flat(lambda g: g.embedding_names())

    def embedding_names_per_rank(self) -> List[List[str]]:
        return self._per_rank(lambda g: g.embedding_names())

    def embedding_shard_metadata(self) -> List[Optional[ShardMetadata]]:
        return self._flat(lambda g: g.embedding_shard_metadata())

    def feature_names(self) -> List[str]:
        return self._flat(lambda g: g.feature_names())

    def embedding_tables(self) -> List[ShardedEmbeddingTable]:
        return self._flat(lambda g: g.embedding_tables)

    def feature_names_per_rank(self) -> List[List[str]]:
        return self._per_rank(lambda g: g.feature_names())

    def features_per_rank(self) -> List[int]:
        return [sum(g.num_features() for g in groups) for groups in self._grouped_embedding_configs_per_rank]

    def _codecs(self, op_name: str) -> Optional[QuantizedCommCodecs]:
        reg = self.qcomm_codecs_registry
        return reg.get(op_name, None) if reg else None
