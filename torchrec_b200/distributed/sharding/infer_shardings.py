"""Sharding strategies of sharded INFERENCE: one process drives every device, the tables are quantized, nothing is trained.

Each strategy reuses the placement logic of its training counterpart (which table shard sits on which device) and swaps the
three stages for single-process ones: the input distribution cuts the request by feature (or buckets ids by row block) and copies
the pieces to their devices, the lookup is the all-device grouped lookup of ``infer_embedding_lookup``, and the output distribution
brings the per-device results to one device (concatenated, summed, or kept as a list for sequences).
Counterpart of the ``Infer*`` classes in ``torchrec/distributed/sharding/{tw,rw,cw}_sharding.py`` and ``{tw,rw,cw}_sequence_sharding.py``."""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch

from torchrec_b200.distributed.dist_data import EmbeddingsAllToOne, KJTOneToAll, SeqEmbeddingsAllToOne
from torchrec_b200.distributed.embedding_sharding import BaseEmbeddingDist, BaseSparseFeaturesDist, EmbeddingShardingInfo, bucketize_kjt_before_all2all
from torchrec_b200.distributed.embedding_types import BaseEmbeddingLookup, InputDistOutputs
from torchrec_b200.distributed.sharding.cw_sharding import BaseCwEmbeddingSharding, PermutePooledEmbeddingsSplit
from torchrec_b200.distributed.sharding.rw_sharding import BaseRwEmbeddingSharding, InferRwPooledEmbeddingDist
from torchrec_b200.distributed.sharding.sequence_sharding import InferSequenceShardingContext
from torchrec_b200.distributed.sharding.tw_sharding import BaseTwEmbeddingSharding, InferTwPooledEmbeddingDist, InferTwSparseFeaturesDist
from torchrec_b200.distributed.types import NullShardingContext, QuantizedCommCodecs, ShardingEnv, ShardingType
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


# ---- output distributions -------------------------------------------------------------------------------------------------
class InferTwSequenceEmbeddingDist(BaseEmbeddingDist[InferSequenceShardingContext, List[torch.Tensor], List[torch.Tensor]]):
    """Per-device rows ``[ids of that device's features, D]`` moved to one device, kept as a list (one entry per device)."""

    def __init__(self, device: torch.device, world_size: int) -> None:
        super().__init__()
        self._dist = SeqEmbeddingsAllToOne(device, world_size)

    def forward(self, local_embs: List[torch.Tensor], sharding_ctx: Optional[InferSequenceShardingContext] = None) -> List[torch.Tensor]:
        return self._dist(local_embs)


InferCwSequenceEmbeddingDist = InferTwSequenceEmbeddingDist
InferRwSequenceEmbeddingDist = InferTwSequenceEmbeddingDist  # the caller restores the request order with the context's permutation


class InferCwPooledEmbeddingDist(BaseEmbeddingDist[NullShardingContext, List[torch.Tensor], torch.Tensor]):
    """Pooled column shards side by side, in device order."""

    def __init__(self, device: torch.device, world_size: int) -> None:
        super().__init__()
        self._dist = EmbeddingsAllToOne(device, world_size, 1)

    def forward(self, local_embs: List[torch.Tensor], sharding_ctx: Optional[NullShardingContext] = None) -> torch.Tensor:
        return self._dist(local_embs)


class InferCwPooledEmbeddingDistWithPermute(InferCwPooledEmbeddingDist):
    """The same, then the column blocks of every table are put next to each other in column order."""

    def __init__(self, device: torch.device, world_size: int, embedding_dims: List[int], permute: List[int]) -> None:
        super().__init__(device, world_size)
        self._permute = PermutePooledEmbeddingsSplit(embedding_dims, permute, device=device)

    def forward(self, local_embs: List[torch.Tensor], sharding_ctx: Optional[NullShardingContext] = None) -> torch.Tensor:
        return self._permute(super().forward(local_embs, sharding_ctx))


# ---- input distributions ----------------------------------------------------------------------------------------------------
class InferRwSparseFeaturesDist(BaseSparseFeaturesDist[InputDistOutputs]):
    """Ids bucketized by row block, bucket ``r`` copied to device ``r``; for sequences the permutation back to request order is
    part of the output."""

    def __init__(self, world_size: int, num_features: int, feature_hash_sizes: List[int], device: Optional[torch.device] = None,
                 is_sequence: bool = False, has_feature_processor: bool = False, need_pos: bool = False,
                 feature_total_num_buckets: Optional[List[int]] = None, keep_original_indices: bool = False) -> None:
        super().__init__()
        self._world_size, self._num_features = world_size, num_features
        div = feature_total_num_buckets if feature_total_num_buckets is not None else [world_size] * len(feature_hash_sizes)
        self.register_buffer("_feature_block_sizes_tensor", torch.tensor([(h + d - 1) // d for h, d in zip(feature_hash_sizes, div)], dtype=torch.int64),
                             persistent=False)
        self._total_blocks = None if feature_total_num_buckets is None else torch.tensor(feature_total_num_buckets, dtype=torch.int64)
        self._dist = KJTOneToAll(splits=[num_features] * world_size, world_size=world_size, device=device)
        self._is_sequence, self._has_feature_processor, self._need_pos = is_sequence, has_feature_processor, need_pos
        self._keep_original_indices = keep_original_indices

    def forward(self, sparse_features: KeyedJaggedTensor) -> InputDistOutputs:
        dev = sparse_features.values().device
        bucketized, permute = bucketize_kjt_before_all2all(
            sparse_features, num_buckets=self._world_size, block_sizes=self._feature_block_sizes_tensor.to(dev),
            total_num_blocks=None if self._total_blocks is None else self._total_blocks.to(dev), output_permute=self._is_sequence,
            bucketize_pos=self._has_feature_processor if sparse_features.weights_or_none() is None else self._need_pos,
            keep_original_indices=self._keep_original_indices)
        return InputDistOutputs(features=self._dist(bucketized).wait(), unbucketize_permute_tensor=permute)


# ---- the strategies ---------------------------------------------------------------------------------------------------------
class _InferStages:
    """Lookup factory shared by all inference strategies; ``_pooled`` picks the lookup, the subclasses add their distributions."""

    _pooled = True

    def create_lookup(self, device: Optional[torch.device] = None, fused_params: Optional[Dict[str, Any]] = None, feature_processor=None) -> BaseEmbeddingLookup:
        from torchrec_b200.distributed.infer_embedding_lookup import InferGroupedEmbeddingsLookup, InferGroupedPooledEmbeddingsLookup

        cls = InferGroupedPooledEmbeddingsLookup if self._pooled else InferGroupedEmbeddingsLookup
        return cls(self._grouped_embedding_configs_per_rank, self._world_size, fused_params, device if device is not None else self._device)

    def _out_device(self, device: Optional[torch.device]) -> torch.device:
        device = device if device is not None else self._device
        return device if device is not None else torch.device("cpu")


class _InferKeySplit(_InferStages):
    def create_input_dist(self, device: Optional[torch.device] = None) -> InferTwSparseFeaturesDist:
        return InferTwSparseFeaturesDist(self.features_per_rank(), self._world_size, device if device is not None else self._device)


class InferTwEmbeddingSharding(_InferKeySplit, BaseTwEmbeddingSharding[NullShardingContext, InputDistOutputs, List[torch.Tensor], torch.Tensor]):
    sharding_type = ShardingType.TABLE_WISE

    def create_output_dist(self, device: Optional[torch.device] = None) -> InferTwPooledEmbeddingDist:
        return InferTwPooledEmbeddingDist(self._out_device(device), self._world_size)


class InferTwSequenceEmbeddingSharding(_InferKeySplit, BaseTwEmbeddingSharding[InferSequenceShardingContext, InputDistOutputs, List[torch.Tensor], List[torch.Tensor]]):
    sharding_type = ShardingType.TABLE_WISE
    _pooled = False

    def create_output_dist(self, device: Optional[torch.device] = None) -> InferTwSequenceEmbeddingDist:
        return InferTwSequenceEmbeddingDist(self._out_device(device), self._world_size)


class InferCwPooledEmbeddingSharding(_InferKeySplit, BaseCwEmbeddingSharding[NullShardingContext, InputDistOutputs, List[torch.Tensor], torch.Tensor]):
    sharding_type = ShardingType.COLUMN_WISE

    def create_output_dist(self, device: Optional[torch.device] = None) -> InferCwPooledEmbeddingDist:
        device = self._out_device(device)
        if self._permute_embeddings and self._embedding_order != list(range(len(self._embedding_order))):
            return InferCwPooledEmbeddingDistWithPermute(device, self._world_size, self._embedding_dims, self._embedding_order)
        return InferCwPooledEmbeddingDist(device, self._world_size)


class InferCwSequenceEmbeddingSharding(_InferKeySplit, BaseCwEmbeddingSharding[InferSequenceShardingContext, InputDistOutputs, List[torch.Tensor], List[torch.Tensor]]):
    sharding_type = ShardingType.COLUMN_WISE
    _pooled = False

    def create_output_dist(self, device: Optional[torch.device] = None) -> InferTwSequenceEmbeddingDist:
        return InferCwSequenceEmbeddingDist(self._out_device(device), self._world_size)


class _InferRowBuckets(_InferStages):
    _sequence = False

    def create_input_dist(self, device: Optional[torch.device] = None) -> InferRwSparseFeaturesDist:
        return InferRwSparseFeaturesDist(
            self._world_size, self._get_num_features(), self._get_feature_hash_sizes(), device if device is not None else self._device,
            is_sequence=self._sequence, has_feature_processor=self._has_feature_processor, need_pos=self._need_pos,
            feature_total_num_buckets=self._get_feature_total_num_buckets())


class InferRwPooledEmbeddingSharding(_InferRowBuckets, BaseRwEmbeddingSharding[NullShardingContext, InputDistOutputs, List[torch.Tensor], torch.Tensor]):
    sharding_type = ShardingType.ROW_WISE

    def create_output_dist(self, device: Optional[torch.device] = None) -> InferRwPooledEmbeddingDist:
        return InferRwPooledEmbeddingDist(self._out_device(device), self._world_size)


class InferRwSequenceEmbeddingSharding(_InferRowBuckets, BaseRwEmbeddingSharding[InferSequenceShardingContext, InputDistOutputs, List[torch.Tensor], List[torch.Tensor]]):
    sharding_type = ShardingType.ROW_WISE
    _pooled = False
    _sequence = True

    def create_output_dist(self, device: Optional[torch.device] = None) -> InferTwSequenceEmbeddingDist:
        return InferRwSequenceEmbeddingDist(self._out_device(device), self._world_size)
