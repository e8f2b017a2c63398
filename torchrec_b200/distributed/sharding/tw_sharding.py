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
    """Whole-table placement; the column-wise shardings reuse everything and only say where the column blocks go."""

    _shard_type = ShardingType.TABLE_WISE

    def _placements(self, info: EmbeddingShardingInfo):
        """``(rank, shard metadata, columns)`` of every shard of one table: here the table itself."""
        yield info.param_sharding.ranks[0], info.param_sharding.sharding_spec.shards[0], info.embedding_config.embedding_dim

    def _shard(self, sharding_infos: List[EmbeddingShardingInfo]) -> List[List[ShardedEmbeddingTable]]:
        per_rank: List[List[ShardedEmbeddingTable]] = [[] for _ in range(self._world_size)]
        for info in sharding_infos:
            cfg = info.embedding_config
            rows = cfg.num_embeddings if cfg.num_embeddings_post_pruning is None else cfg.num_embeddings_post_pruning
            whole = global_metadata_of(info)
            for rank, shard, cols in self._placements(info):
                per_rank[self._remap(rank, self._shard_type)].append(make_sharded_table(info, shard, whole, rows, cols))
        return per_rank


class TwSparseFeaturesDist(BaseSparseFeaturesDist[KeyedJaggedTensor]):
    """Ids travel by feature: rank r receives, for the whole global batch, the features of the tables it holds."""

    def __init__(self, pg: dist.ProcessGroup, features_per_rank: List[int]) -> None:
        super().__init__()
        self._dist = KJTAllToAll(pg=pg, splits=features_per_rank)

    def forward(self, sparse_features: KeyedJaggedTensor) -> Awaitable[Awaitable[KeyedJaggedTensor]]:
        return self._dist(sparse_features)


class TwPooledEmbeddingDist(BaseEmbeddingDist[EmbeddingShardingContext, torch.Tensor, torch.Tensor]):
    """Pooled rows ``[B_global, D_local]`` to ``[B_local, sum D]``.  The exchange module is built on first use: the fixed-batch
    all-to-all, or the variable-batch one when the first context says that features differ in batch size."""

    def __init__(self, pg: dist.ProcessGroup, dim_sum_per_rank: List[int], emb_dim_per_rank_per_feature: List[List[int]],
                 device: Optional[torch.device] = None, callbacks: Optional[List[Callable[[torch.Tensor], torch.Tensor]]] = None,
                 qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None) -> None:
        super().__init__()
        codecs = (qcomm_codecs_registry or {}).get(CommOp.POOLED_EMBEDDINGS_ALL_TO_ALL.name)
        self._build_fixed = lambda: PooledEmbeddingsAllToAll(pg=pg, dim_sum_per_rank=dim_sum_per_rank, device=device, callbacks=callbacks, codecs=codecs)
        self._build_variable = lambda: VariableBatchPooledEmbeddingsAllToAll(pg=pg, emb_dim_per_rank_per_feature=emb_dim_per_rank_per_feature,
                                                                             device=device, codecs=codecs)
        self._dist: Optional[PooledEmbeddingsAllToAll] = None
        self._variable_dist: Optional[VariableBatchPooledEmbeddingsAllToAll] = None

    def forward(self, local_embs: torch.Tensor, sharding_ctx: Optional[EmbeddingShardingContext] = None) -> Awaitable[torch.Tensor]:
        if sharding_ctx is not None and sharding_ctx.variable_batch_per_feature:
            if self._variable_dist is None:
                self._variable_dist = self._build_variable()
            return self._variable_dist(local_embs, batch_size_per_rank_per_feature=sharding_ctx.batch_size_per_rank_per_feature,
                                       batch_size_per_feature_pre_a2a=sharding_ctx.batch_size_per_feature_pre_a2a)
        if self._dist is None:
            self._dist = self._build_fixed()
        if sharding_ctx is None:
            return self._dist(local_embs)
        return self._dist(local_embs, batch_size_per_rank=sharding_ctx.batch_size_per_rank or None)


class _KeySplitPooledRouting:
    """Input distribution, lookup and output distribution of the pooled shardings that route ids by feature (table-wise and the
    column-wise family); ``_output_callbacks`` lets a sharding post-process the exchanged rows."""

    def _output_callbacks(self, device: Optional[torch.device]) -> Optional[List[Callable[[torch.Tensor], torch.Tensor]]]:
        return None

    def create_input_dist(self, device: Optional[torch.device] = None) -> TwSparseFeaturesDist:
        assert self._pg is not None
        return TwSparseFeaturesDist(self._pg, self.features_per_rank())

    def create_lookup(self, device: Optional[torch.device] = None, fused_params: Optional[Dict[str, Any]] = None, feature_processor=None) -> BaseEmbeddingLookup:
        return GroupedPooledEmbeddingsLookup(grouped_configs=self._grouped_embedding_configs, pg=self._pg, device=device if device is not None else self._device,
                                             feature_processor=feature_processor, sharding_type=self._shard_type)

    def create_output_dist(self, device: Optional[torch.device] = None) -> TwPooledEmbeddingDist:
        assert self._pg is not None
        device = device if device is not None else self._device
        return TwPooledEmbeddingDist(pg=self._pg, dim_sum_per_rank=self._dim_sum_per_rank(), emb_dim_per_rank_per_feature=self._emb_dim_per_rank_per_feature(),
                                     device=device, callbacks=self._output_callbacks(device), qcomm_codecs_registry=self.qcomm_codecs_registry)


class TwPooledEmbeddingSharding(_KeySplitPooledRouting, BaseTwEmbeddingSharding[EmbeddingShardingContext, KeyedJaggedTensor, torch.Tensor, torch.Tensor]):
    sharding_type = ShardingType.TABLE_WISE


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


_INFER_NAMES = ("InferTwEmbeddingSharding",)


def __getattr__(name: str):
    """The inference strategies live in ``infer_shardings`` (they build on every training strategy); they are reachable from
    here under the reference's import path."""
    if name in _INFER_NAMES:
        from torchrec_b200.distributed.sharding import infer_shardings

        return getattr(infer_shardings, name)
    raise AttributeError(name)
