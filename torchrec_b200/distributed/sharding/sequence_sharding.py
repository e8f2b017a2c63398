"""Context and base output dist of the sequence (unpooled) shardings
(cf. ``torchrec/distributed/sharding/sequence_sharding.py``)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from torchrec_b200.distributed.embedding_sharding import EmbeddingShardingContext
from torchrec_b200.distributed.embedding_types import KJTList
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
