"""Data-parallel sequence embeddings: local lookup of the local batch
(cf. ``torchrec/distributed/sharding/dp_sequence_sharding.py``)."""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch

from torchrec_b200.distributed.embedding_lookup import GroupedEmbeddingsLookup
from torchrec_b200.distributed.embedding_sharding import BaseEmbeddingDist, BaseSparseFeaturesDist
from torchrec_b200.distributed.embedding_types import BaseEmbeddingLookup
from torchrec_b200.distributed.sharding.dp_sharding import BaseDpEmbeddingSharding, DpSparseFeaturesDist
from torchrec_b200.distributed.sharding.sequence_sharding import SequenceShardingContext
from torchrec_b200.distributed.types import Awaitable, NoWait, ShardingType
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class DpSequenceEmbeddingDist(BaseEmbeddingDist[SequenceShardingContext, torch.Tensor, torch.Tensor]):
    def forward(self, local_embs: torch.Tensor, sharding_ctx: Optional[SequenceShardingContext] = None) -> Awaitable[torch.Tensor]:
        return NoWait(local_embs)


class DpSequenceEmbeddingSharding(BaseDpEmbeddingSharding[SequenceShardingContext, KeyedJaggedTensor, torch.Tensor, torch.Tensor]):
    sharding_type = ShardingType.DATA_PARALLEL

    def create_input_dist(self, device: Optional[torch.device] = None) -> BaseSparseFeaturesDist[KeyedJaggedTensor]:
        return DpSparseFeaturesDist()

    def create_lookup(self, device: Optional[torch.device] = None, fused_params: Optional[Dict[str, Any]] = None, feature_processor=None) -> BaseEmbeddingLookup:
        assert feature_processor is None
        return GroupedEmbeddingsLookup(grouped_configs=self._grouped_embedding_configs, pg=self._env.process_group, device=device if device is not None else self._device)

    def create_output_dist(self, device: Optional[torch.device] = None) -> BaseEmbeddingDist[SequenceShardingContext, torch.Tensor, torch.Tensor]:
        return DpSequenceEmbeddingDist()
