"""Table-wise sharding of unpooled (sequence) embeddings: whole tables live on one rank; ids travel there by a key split and the
rows come back by the sequence all-to-all (cf. ``torchrec/distributed/sharding/tw_sequence_sharding.py``)."""
from __future__ import annotations

from typing import Optional

import torch

from torchrec_b200.distributed.sharding.sequence_sharding import SequenceLookupMixin, SequenceRowsReturn, SequenceShardingContext
from torchrec_b200.distributed.sharding.tw_sharding import BaseTwEmbeddingSharding, TwSparseFeaturesDist
from torchrec_b200.distributed.types import ShardingType
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class TwSequenceEmbeddingDist(SequenceRowsReturn):
    """The rows' way back for table-wise (and column-wise) shards: no bucketization to undo."""

    def __init__(self, pg, features_per_rank, device=None, qcomm_codecs_registry=None) -> None:
        super().__init__(pg, features_per_rank, device, qcomm_codecs_registry, restore_order=False)


class _KeySplitSequenceRouting(SequenceLookupMixin):
    """Ids are routed by feature (every rank receives the features of the tables it holds)."""

    def create_input_dist(self, device: Optional[torch.device] = None) -> TwSparseFeaturesDist:
        assert self._pg is not None
        return TwSparseFeaturesDist(self._pg, self.features_per_rank())

    def create_output_dist(self, device: Optional[torch.device] = None) -> TwSequenceEmbeddingDist:
        assert self._pg is not None
        return TwSequenceEmbeddingDist(self._pg, self.features_per_rank(), device if device is not None else self._device, self.qcomm_codecs_registry)


class TwSequenceEmbeddingSharding(_KeySplitSequenceRouting, BaseTwEmbeddingSharding[SequenceShardingContext, KeyedJaggedTensor, torch.Tensor, torch.Tensor]):
    sharding_type = ShardingType.TABLE_WISE


_INFER_NAMES = ("InferTwSequenceEmbeddingDist", "InferTwSequenceEmbeddingSharding")


def __getattr__(name: str):
    """The inference strategies live in ``infer_shardings`` (they build on every training strategy); they are reachable from
    here under the reference's import path."""
    if name in _INFER_NAMES:
        from torchrec_b200.distributed.sharding import infer_shardings

        return getattr(infer_shardings, name)
    raise AttributeError(name)
