"""Column-wise sharding of sequence embeddings: each column shard acts as a table-wise table and the
per-shard rows are concatenated along the embedding dim when the output is assembled
(cf. ``torchrec/distributed/sharding/cw_sequence_sharding.py``)."""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch

from torchrec_b200.distributed.embedding_lookup import GroupedEmbeddingsLookup
from torchrec_b200.distributed.embedding_sharding import BaseEmbeddingDist, BaseSparseFeaturesDist
from torchrec_b200.distributed.embedding_types import BaseEmbeddingLookup
from torchrec_b200.distributed.sharding.cw_sharding import BaseCwEmbeddingSharding
from torchrec_b200.distributed.sharding.sequence_sharding import SequenceShardingContext
from torchrec_b200.distributed.sharding.tw_sequence_sharding import TwSequenceEmbeddingDist
from torchrec_b200.distributed.sharding.tw_sharding import TwSparseFeaturesDist
from torchrec_b200.distributed.types import ShardingType
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class CwSequenceEmbeddingSharding(BaseCwEmbeddingSharding[SequenceShardingContext, KeyedJaggedTensor, torch.Tensor, torch.Tensor]):
    sharding_type = ShardingType.COLUMN_WISE

    def create_input_dist(self, device: Optional[torch.device] = None) -> BaseSparseFeaturesDist[KeyedJaggedTensor]:
        assert self._pg is not None
        return TwSparseFeaturesDist(self._pg, self.features_per_rank())

    def create_lookup(self, device: Optional[torch.device] = None, fused_params: Optional[Dict[str, Any]] = None, feature_processor=None) -> BaseEmbeddingLookup:
        assert feature_processor is None
        return GroupedEmbeddingsLookup(grouped_configs=self._grouped_embedding_configs, pg=self._pg, device=device if device is not None else self._device)

    def create_output_dist(self, device: Optional[torch.device] = None) -> BaseEmbeddingDist[SequenceShardingContext, torch.Tensor, torch.Tensor]:
        assert self._pg is not None
        return TwSequenceEmbeddingDist(self._pg, self.features_per_rank(), device if device is not None else self._device, qcomm_codecs_registry=self.qcomm_codecs_registry)
