"""What all sequence (unpooled) shardings share: the context that carries the input distribution's routes to the output
distribution, the output distribution itself (rows travel back along the routes their ids came by) and the lookup factory.
The per-type modules (``tw_/cw_/rw_/dp_sequence_sharding.py``) only say how ids are routed.
(cf. ``torchrec/distributed/sharding/sequence_sharding.py`` and the ``*_sequence_sharding.py`` files next to it.)"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from torchrec_b200.distributed.embedding_sharding import BaseEmbeddingDist, EmbeddingShardingContext
from torchrec_b200.distributed.embedding_types import BaseEmbeddingLookup, KJTList
from torchrec_b200.distributed.types import Awaitable, CommOp, NoWait, QuantizedCommCodecs
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor
from torchrec_b200.streamable import Multistreamable


class SequenceShardingContext(EmbeddingShardingContext):
    """What the sequence output all-to-all needs from the input dist: the splits of the ``values``
    all-to-all (rows come back along the same routes), the recat used after it, the lengths after it and,
    for row-wise, the permutation that restores the original id order."""

    def __init__(self, batch_size_per_rank: Optional[List[int]] = None, batch_size_per_rank_per_feature: Optional[List[List[int]]] = None,
                 batch_size_per_feature_pre_a2a: Optional[List[int]] = None, variable_batch_per_feature: bool = False,
                 features_before_input_dist: Optional[KeyedJaggedTensor] = None, input_splits: Optional[List[int]] = None,
                 output_splits: Optional[List[int]] = None, sparse_features_recat: Optional[torch.Tensor] = None,
                 unbucketize_permute_tensor: Optional[torch.Tensor] = None, lengths_after_input_dist: Optional[torch.Tensor] = None) -> None:
        super().__init__(batch_size_per_rank, batch_size_per_rank_per_feature, batch_size_per_feature_pre_a2a, variable_batch_per_feature)
        self.features_before_input_dist = features_before_input_dist
        self.input_splits: List[int] = input_splits if input_splits is not None else []
        self.output_splits: List[int] = output_splits if output_splits is not None else []
        self.sparse_features_recat = sparse_features_recat
        self.unbucketize_permute_tensor = unbucketize_permute_tensor
        self.lengths_after_input_dist = lengths_after_input_dist

    def record_stream(self, stream: torch.Stream) -> None:
        if self.features_before_input_dist is not None:
            self.features_before_input_dist.record_stream(stream)
        for t in (self.sparse_features_recat, self.unbucketize_permute_tensor, self.lengths_after_input_dist):
            if t is not None and t.is_cuda:
                t.record_stream(stream)


@dataclass
class InferSequenceShardingContext(Multistreamable):
    features: KJTList
    features_before_input_dist: Optional[KeyedJaggedTensor] = None
    unbucketize_permute_tensor: Optional[torch.Tensor] = None
    bucket_mapping_tensor: Optional[torch.Tensor] = None
    bucketized_length: Optional[torch.Tensor] = None
    embedding_names_per_rank: Optional[List[List[str]]] = None

    def record_stream(self, stream: torch.Stream) -> None:
        for f in self.features:
            f.record_stream(stream)
        if self.features_before_input_dist is not None:
            self.features_before_input_dist.record_stream(stream)
        for t in (self.unbucketize_permute_tensor, self.bucket_mapping_tensor, self.bucketized_length):
            if t is not None and t.is_cuda:
                t.record_stream(stream)


class SequenceRowsReturn(BaseEmbeddingDist[SequenceShardingContext, torch.Tensor, torch.Tensor]):
    """Output distribution of every sharded sequence lookup: the rows ``[sum L, D]`` go back to the ranks that sent the ids, along
    the splits recorded by the input distribution.  ``restore_order`` additionally undoes the row-wise bucketization."""

    def __init__(self, pg: dist.ProcessGroup, features_per_rank: List[int], device: Optional[torch.device] = None,
                 qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None, restore_order: bool = False) -> None:
        super().__init__()
        from torchrec_b200.distributed.dist_data import SequenceEmbeddingsAllToAll

        codecs = (qcomm_codecs_registry or {}).get(CommOp.SEQUENCE_EMBEDDINGS_ALL_TO_ALL.name)
        self._dist = SequenceEmbeddingsAllToAll(pg, features_per_rank, device, codecs=codecs)
        self._restore_order = restore_order

    def forward(self, local_embs: torch.Tensor, sharding_ctx: Optional[SequenceShardingContext] = None) -> Awaitable[torch.Tensor]:
        assert sharding_ctx is not None, "the sequence output distribution needs the routes of the input distribution"
        c = sharding_ctx
        return self._dist(local_embs, lengths=c.lengths_after_input_dist, input_splits=c.input_splits, output_splits=c.output_splits,
                          batch_size_per_rank=c.batch_size_per_rank, sparse_features_recat=c.sparse_features_recat,
                          unbucketize_permute_tensor=c.unbucketize_permute_tensor if self._restore_order else None)


class LocalRows(BaseEmbeddingDist[SequenceShardingContext, torch.Tensor, torch.Tensor]):
    """Output 'distribution' of a replicated table: the rows are already where they are wanted."""

    def forward(self, local_embs: torch.Tensor, sharding_ctx: Optional[SequenceShardingContext] = None) -> Awaitable[torch.Tensor]:
        return NoWait(local_embs)


class SequenceLookupMixin:
    """``create_lookup`` of the sequence shardings: the grouped unpooled lookup over this rank's shards."""

    def create_lookup(self, device: Optional[torch.device] = None, fused_params: Optional[Dict[str, Any]] = None, feature_processor=None) -> BaseEmbeddingLookup:
        from torchrec_b200.distributed.embedding_lookup import GroupedEmbeddingsLookup

        pg = getattr(self, "_pg", None)
        if pg is None:
            pg = self._env.process_group
        return GroupedEmbeddingsLookup(grouped_configs=self._grouped_embedding_configs, pg=pg, device=device if device is not None else self._device)
