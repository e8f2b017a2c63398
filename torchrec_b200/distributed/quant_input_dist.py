"""Input distribution of sharded quantized modules.  One process drives every device, so "distribution" means: cut the features
of every device's tables out of the request and copy them to that device (table-wise and column-wise placement), and bucketize the
ids of row-wise tables by row block, one bucket per device.  ``ShardedQuantEbcInputDist`` serves the pooled collection,
``ShardedQuantEcInputDist`` the sequence collection (it also returns the permutation that puts looked-up rows back in request
order).  Counterpart of ``torchrec/distributed/quant_embeddingbag.py:576`` and ``torchrec/distributed/quant_embedding.py:1067``."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Hashable, List, Optional

import torch
from torch import nn

from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


def device_of_rank(rank: int, device_type: str) -> torch.device:
    return torch.device("cuda", rank) if device_type == "cuda" else torch.device(device_type)


@dataclass
class QuantInputDistOutputs:
    table_wise: Dict[int, KeyedJaggedTensor] = field(default_factory=dict)        # rank -> features of its whole tables, on its device
    column_wise: Dict[Hashable, KeyedJaggedTensor] = field(default_factory=dict)  # shard key -> features of its column shards, on its device
    row_wise: List[KeyedJaggedTensor] = field(default_factory=list)               # per rank: the bucket of that rank, on its device
    row_wise_request: Optional[KeyedJaggedTensor] = None                          # the row-wise features as they came (request order)
    unbucketize_permute: Optional[torch.Tensor] = None                            # sequence form: bucketized position of every request id


class _ShardedQuantInputDist(nn.Module):
    _restore_order = False

    def __init__(self, world_size: int, device_type: str, table_wise_features: Dict[int, List[str]], column_wise_features: Dict[Hashable, List[str]],
                 column_wise_rank: Dict[Hashable, int], row_wise_features: List[str], row_wise_block_sizes: torch.Tensor) -> None:
        super().__init__()
        self._world_size, self._device_type = world_size, device_type
        self._tw = {r: list(f) for r, f in table_wise_features.items() if f}
        self._cw = {k: list(f) for k, f in column_wise_features.items() if f}
        self._cw_rank = dict(column_wise_rank)
        self._rw = list(row_wise_features)
        self.register_buffer("_rw_block_sizes", row_wise_block_sizes.to(torch.int64), persistent=False)

    def _cut(self, features: KeyedJaggedTensor, keys: List[str], names: List[str], rank: int) -> KeyedJaggedTensor:
        return features.permute([keys.index(f) for f in names]).to(device_of_rank(rank, self._device_type), non_blocking=True)

    def forward(self, features: KeyedJaggedTensor) -> QuantInputDistOutputs:
        from torchrec_b200.distributed.embedding_sharding import bucketize_kjt_before_all2all

        keys = features.keys()
        out = QuantInputDistOutputs()
        for rank, names in self._tw.items():
            out.table_wise[rank] = self._cut(features, keys, names, rank)
        for key, names in self._cw.items():
            out.column_wise[key] = self._cut(features, keys, names, self._cw_rank[key])
        if self._rw:
            request = features.permute([keys.index(f) for f in self._rw])
            bucketized, permute = bucketize_kjt_before_all2all(request, num_buckets=self._world_size,
                                                               block_sizes=self._rw_block_sizes.to(request.values().device), output_permute=self._restore_order)
            for rank, part in enumerate(bucketized.split([len(self._rw)] * self._world_size)):
                local = KeyedJaggedTensor(keys=self._rw, values=part.values(), weights=part.weights_or_none(), lengths=part.lengths(), stride=features.stride())
                out.row_wise.append(local.to(device_of_rank(rank, self._device_type), non_blocking=True))
            out.row_wise_request, out.unbucketize_permute = request, permute
        return out


class ShardedQuantEbcInputDist(_ShardedQuantInputDist):
    """Pooled collection: no order to restore, bags are summed over the devices."""


class ShardedQuantEcInputDist(_ShardedQuantInputDist):
    """Sequence collection: looked-up rows come back in (device, feature, sample) order; ``unbucketize_permute`` undoes that."""

    _restore_order = True


# ---- choosing the inference strategy of a group of tables ---------------------------------------------------------------------
def get_device_from_parameter_sharding(ps) -> Any:
    """Device type of a table's shards: one string, or a tuple (one entry per shard) when a row-wise table is spread over device types."""
    shards = getattr(ps.sharding_spec, "shards", None)
    if shards is None:
        raise ValueError("Expected EnumerableShardingSpec as input to the function")
    kinds = tuple(str(s.placement).split("/")[-1].split(":")[0] for s in shards)
    if len(set(kinds)) == 1:
        return kinds[0]
    assert ps.sharding_type == "row_wise", "Only row_wise sharding supports sharding across multiple device types for a table"
    return kinds


def get_device_from_sharding_infos(emb_shard_infos) -> Any:
    kinds = {get_device_from_parameter_sharding(info.param_sharding) for info in emb_shard_infos}
    assert len(kinds) == 1, "All shards should be on the same type of device"
    return next(iter(kinds))


def get_device_for_first_shard_from_sharding_infos(emb_shard_infos) -> str:
    kind = get_device_from_sharding_infos(emb_shard_infos)
    return kind[0] if isinstance(kind, tuple) else kind


def create_infer_embedding_bag_sharding(sharding_type: str, sharding_infos, env, device: Optional[torch.device] = None):
    """The pooled inference strategy for ``sharding_type`` (table-wise, row-wise or column-wise)."""
    from torchrec_b200.distributed.sharding import infer_shardings as inf
    from torchrec_b200.distributed.types import ShardingType

    if sharding_type == ShardingType.TABLE_WISE.value:
        return inf.InferTwEmbeddingSharding(sharding_infos, env, device)
    if sharding_type == ShardingType.ROW_WISE.value:
        return inf.InferRwPooledEmbeddingSharding(sharding_infos, env, device)
    if sharding_type == ShardingType.COLUMN_WISE.value:
        return inf.InferCwPooledEmbeddingSharding(sharding_infos, env, device, permute_embeddings=True)
    raise ValueError(f"Sharding type not supported {sharding_type}")


def create_infer_embedding_sharding(sharding_type: str, sharding_infos, env, device: Optional[torch.device] = None):
    """The sequence inference strategy for ``sharding_type``."""
    from torchrec_b200.distributed.sharding import infer_shardings as inf
    from torchrec_b200.distributed.types import ShardingType

    if sharding_type == ShardingType.TABLE_WISE.value:
        return inf.InferTwSequenceEmbeddingSharding(sharding_infos, env, device)
    if sharding_type == ShardingType.ROW_WISE.value:
        return inf.InferRwSequenceEmbeddingSharding(sharding_infos, env, device)
    if sharding_type == ShardingType.COLUMN_WISE.value:
        return inf.InferCwSequenceEmbeddingSharding(sharding_infos, env, device)
    raise ValueError(f"Sharding type not supported {sharding_type}")


def flatten_feature_lengths(features: KeyedJaggedTensor) -> KeyedJaggedTensor:
    return features.flatten_lengths() if features.lengths().dim() > 1 else features
