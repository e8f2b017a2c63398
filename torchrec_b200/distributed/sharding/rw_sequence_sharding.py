"""Row-wise sharding of sequence embeddings: ids are bucketized by row block and looked up on the owning rank; the rows return by
the sequence all-to-all and are put back in the order of the original ids
(cf. ``torchrec/distributed/sharding/rw_sequence_sharding.py``)."""
from __future__ import annotations

from typing import Optional

import torch

from torchrec_b200.distributed.sharding.rw_sharding import BaseRwEmbeddingSharding, RwSparseFeaturesDist
from torchrec_b200.distributed.sharding.sequence_sharding import SequenceLookupMixin, SequenceRowsReturn, SequenceShardingContext
from torchrec_b200.distributed.types import ShardingType
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class RwSequenceEmbeddingDist(SequenceRowsReturn):
    """The rows' way back for row-wise shards: every rank serves all features, and the bucketization is undone at the end."""

    def __init__(self, pg, num_features: int, device=None, qcomm_codecs_registry=None) -> None:
        super().__init__(pg, [num_features] * pg.size(), device, qcomm_codecs_registry, restore_order=True)


class RwSequenceEmbeddingSharding(SequenceLookupMixin, BaseRwEmbeddingSharding[SequenceShardingContext, KeyedJaggedTensor, torch.Tensor, torch.Tensor]):
    sharding_type = ShardingType.ROW_WISE

    def create_input_dist(self, device: Optional[torch.device] = None) -> RwSparseFeaturesDist:
        return RwSparseFeaturesDist(
            pg=self._pg, num_features=self._get_num_features(), feature_hash_sizes=self._get_feature_hash_sizes(),
            feature_total_num_buckets=self._get_feature_total_num_buckets(), device=device if device is not None else self._device,
            is_sequence=True, has_feature_processor=self._has_feature_processor, need_pos=False,
            keep_original_indices=getattr(self, "_keep_original_indices", False))

    def create_output_dist(self, device: Optional[torch.device] = None) -> RwSequenceEmbeddingDist:
        return RwSequenceEmbeddingDist(self._pg, self._get_num_features(), device if device is not None else self._device, self.qcomm_codecs_registry)


_INFER_NAMES = ("InferRwSequenceEmbeddingDist", "InferRwSequenceEmbeddingSharding")


def __getattr__(name: str):
    """The inference strategies live in ``infer_shardings`` (they build on every training strategy); they are reachable from
    here under the reference's import path."""
    if name in _INFER_NAMES:
        from torchrec_b200.distributed.sharding import infer_shardings

        return getattr(infer_shardings, name)
    raise AttributeError(name)
