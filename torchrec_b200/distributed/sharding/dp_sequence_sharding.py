"""Data-parallel sequence embeddings: every rank looks its own batch up in its own replica
(cf. ``torchrec/distributed/sharding/dp_sequence_sharding.py``)."""
from __future__ import annotations

from typing import Optional

import torch

from torchrec_b200.distributed.sharding.dp_sharding import BaseDpEmbeddingSharding, DpSparseFeaturesDist
from torchrec_b200.distributed.sharding.sequence_sharding import LocalRows, SequenceLookupMixin, SequenceShardingContext
from torchrec_b200.distributed.types import ShardingType
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

DpSequenceEmbeddingDist = LocalRows


class DpSequenceEmbeddingSharding(SequenceLookupMixin, BaseDpEmbeddingSharding[SequenceShardingContext, KeyedJaggedTensor, torch.Tensor, torch.Tensor]):
    sharding_type = ShardingType.DATA_PARALLEL

    def create_input_dist(self, device: Optional[torch.device] = None) -> DpSparseFeaturesDist:
        return DpSparseFeaturesDist()

    def create_output_dist(self, device: Optional[torch.device] = None) -> LocalRows:
        return LocalRows()
