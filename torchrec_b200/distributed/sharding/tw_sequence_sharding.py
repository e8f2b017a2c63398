"""Table-wise sharding of unpooled (sequence) embeddings
(cf. ``torchrec/distributed/sharding/tw_sequence_sharding.py``)."""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from torchrec_b200.distributed.dist_data import SequenceEmbeddingsAllToAll
from torchrec_b200.distributed.embedding_lookup import GroupedEmbeddingsLookup
from torchrec_b200.distributed.embedding_sharding import BaseEmbeddingDist, BaseSparseFeaturesDist
from torchrec_b200.distributed.embedding_types import BaseEmbeddingLookup
from torchrec_b200.distributed.sharding.sequence_sharding import SequenceShardingContext
from torchrec_b200.distributed.sharding.tw_sharding import BaseTwEmbeddingSharding, TwSparseFeaturesDist
from torchrec_b200.distributed.types import Awaitable, CommOp, QuantizedCommCodecs, ShardingType
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class TwSequenceEmbeddingDist(BaseEmbeddingDist[SequenceShardingContext, torch.Tensor, torch.Tensor]):
    """Rows ``[sum L, D]`` go back to the ranks that sent the ids, along the recorded ``values`` splits."""

    def __init__(self, pg: dist.ProcessGroup, features_per_rank: List[int], device: Optional[torch.device] = None,
                 qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None) -> None:
        super().__init__()
        self._dist = SequenceEmbeddingsAllToAll(
            pg, features_per_rank, device,
            codecs=qcomm_codecs_registry.get(CommOp.SEQUENCE_EMBEDDINGS_ALL_TO_ALL.name, None) if qcomm_codecs_registry else None,
        )

    def forward(self, local_embs: torch.Tensor, sharding_ctx: Optional[SequenceShardingContext] = None) -> Awaitable[torch.Tensor]:
        assert sharding_ctx is not None
        return self._dist(
            local_embs, lengths=sharding_ctx.lengths_after_input_dist, input_splits=sharding_ctx.input_splits,
            output_splits=sharding_ctx.output_splits, batch_size_per_rank=sharding_ctx.batch_size_per_rank,
            sparse_features_recat=sharding_ctx.sparse_features_recat, unbucketize_permute_tensor=None,
        )


class TwSequenceEmbeddingSharding(BaseTwEmbeddingSharding[SequenceShardingContext, KeyedJaggedTensor, torch.Tensor, torch.Tensor]):
    sharding_type = ShardingType.TABLE_WISE

    def create_input_dist(self, device: Optional[torch.device] = None) -> BaseSparseFeaturesDist[KeyedJaggedTensor]:
        assert self._pg is not None
        return TwSparseFeaturesDist(self._pg, self.features_per_rank())

    def create_lookup(self, device: Optional[torch.device] = None, fused_params: Optional[Dict[str, Any]] = None, feature_processor=None) -> BaseEmbeddingLookup:
        assert feature_processor is None
        return GroupedEmbeddingsLookup(grouped_configs=self._grouped_embedding_configs, pg=self._pg, device=device if device is not None else self._device)

    def create_output_dist(self, device: Optional[torch.device] = None) -> BaseEmbeddingDist[SequenceShardingContext, torch.Tensor, torch.Tensor]:
        assert self._pg is not None
        return TwSequenceEmbeddingDist(self._pg, self.features_per_rank(), device if device is not None else self._device, qcomm_codecs_registry=self.qcomm_codecs_registry)
