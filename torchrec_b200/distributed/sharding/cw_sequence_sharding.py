"""Column-wise sharding of sequence embeddings: every column shard is routed like a table-wise table, and the sharded module puts
the shards' rows side by side along the embedding dimension (cf. ``torchrec/distributed/sharding/cw_sequence_sharding.py``)."""
from __future__ import annotations

import torch

from torchrec_b200.distributed.sharding.cw_sharding import BaseCwEmbeddingSharding
from torchrec_b200.distributed.sharding.sequence_sharding import SequenceShardingContext
from torchrec_b200.distributed.sharding.tw_sequence_sharding import _KeySplitSequenceRouting
from torchrec_b200.distributed.types import ShardingType
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class CwSequenceEmbeddingSharding(_KeySplitSequenceRouting, BaseCwEmbeddingSharding[SequenceShardingContext, KeyedJaggedTensor, torch.Tensor, torch.Tensor]):
    sharding_type = ShardingType.COLUMN_WISE


_INFER_NAMES = ("InferCwSequenceEmbeddingSharding", "InferCwSequenceEmbeddingDist")


def __getattr__(name: str):
    """The inference strategies live in ``infer_shardings`` (they build on every training strategy); they are reachable from
    here under the reference's import path."""
    if name in _INFER_NAMES:
        from torchrec_b200.distributed.sharding import infer_shardings

        return getattr(infer_shardings, name)
    raise AttributeError(name)
