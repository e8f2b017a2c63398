"""Row-wise sharding of sequence embeddings: ids are bucketized by row block, looked up on the owning
rank, returned by the sequence all-to-all and put back in their original order
(cf. ``torchrec/distributed/sharding/rw_sequence_sharding.py``)."""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from torchrec_b200.distributed.dist_data import SequenceEmbeddingsAllToAll
from torchrec_b200.distributed.embedding_lookup import GroupedEmbeddingsLookup
from torchrec_b200.distributed.embedding_sharding import BaseEmbeddingDist, BaseSparseFeaturesDist
from torchrec_b200.distributed.embedding_types import BaseEmbeddingLookup
from torchrec_b200.distributed.sharding.rw_sharding import BaseRwEmbeddingSharding, RwSparseFeaturesDist
from torchrec_b200.distributed.sharding.sequence_sharding import SequenceShardingContext
from torchrec_b200.distributed.types import Awaitable, CommOp, QuantizedCommCodecs, ShardingType
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class RwSequenceEmbeddingDist(BaseEmbeddingDist[SequenceShardingContext, torch.Tensor, torch.Tensor]):
    def __init__(self, pg: dist.ProcessGroup, num_features: int, device: Optional[torch.device] = None,
                 qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None) -> None:
        super().__init__()
        self._dist = SequenceEmbeddingsAllToAll(
            pg, [num_features] * pg.size(), device,
            codecs=qcomm_codecs_registry.get(CommOp.SEQUENCE_EMBEDDINGS_ALL_TO_ALL.name, None) if qcomm_codecs_registry else None,
        )

    def forward(self, local_embs: torch.Tensor, sharding_ctx: Optional[SequenceShardingContext] = None) -> Awaitable[torch.Tensor]:
        assert sharding_ctx is not None
        return self._dist(
            local_embs, lengths=sharding_ctx.lengths_after_input_dist, input_splits=sharding_ctx.input_splits,
            output_splits=sharding_ctx.output_splits, batch_size_per_rank=sharding_ctx.batch_size_per_rank,
            sparse_features_recat=sharding_ctx.sparse_features_recat, unbucketize_permute_tensor=sharding_ctx.unbucketize_permute_tensor,
        )


class RwSequenceEmbeddingSharding(BaseRwEmbeddingSharding[SequenceShardingContext, KeyedJaggedTensor, torch.Tensor, torch.Tensor]):
    sharding_type = ShardingType.ROW_WISE

    def create_input_dist(self, device: Optional[torch.device] = None) -> BaseSparseFeaturesDist[KeyedJaggedTensor]:
        return RwSparseFeaturesDist(
            pg=self._pg, num_features=self._get_num_features(), feature_hash_sizes=self._get_feature_hash_sizes(),
            feature_total_num_buckets=self._get_feature_total_num_buckets(), device=device if device is not None else self._device,
            is_sequence=True, has_feature_processor=self._has_feature_processor, need_pos=False,
            keep_original_indices=getattr(self, "_keep_original_indices", False),
        )

    def create_lookup(self, device: Optional[torch.device] = None, fused_params: Optional[Dict[str, Any]] = None, feature_processor=None) -> BaseEmbeddingLookup:
        return GroupedEmbeddingsLookup(grouped_configs=self._grouped_embedding_configs, pg=self._pg, device=device if device is not None else self._device)

    def create_output_dist(self, device: Optional[torch.device] = None) -> BaseEmbeddingDist[SequenceShardingContext, torch.Tensor, torch.Tensor]:
        return RwSequenceEmbeddingDist(self._pg, self._get_num_features(), device if device is not None else self._device, qcomm_codecs_registry=self.qcomm_codecs_registry)
