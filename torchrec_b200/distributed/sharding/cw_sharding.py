"""Column-wise sharding: a table is cut along the embedding dim; every column shard behaves like a
table-wise table on its rank, and the pooled output is re-interleaved so that each feature's
columns are contiguous again.  Counterpart of ``torchrec/distributed/sharding/cw_sharding.py``.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional, Set, Tuple

import torch

from torchrec_b200.distributed.embedding_lookup import GroupedPooledEmbeddingsLookup
from torchrec_b200.distributed.embedding_sharding import (
    BaseEmbeddingDist,
    BaseSparseFeaturesDist,
    EmbeddingShardingContext,
    EmbeddingShardingInfo,
)
from torchrec_b200.distributed.embedding_types import BaseEmbeddingLookup, ShardedEmbeddingTable
from torchrec_b200.distributed.sharding.common import C, F, T, W, global_metadata_of, make_sharded_table
from torchrec_b200.distributed.sharding.tw_sharding import BaseTwEmbeddingSharding, _KeySplitPooledRouting
from torchrec_b200.distributed.types import QuantizedCommCodecs, ShardingEnv, ShardingType, ShardMetadata
from torchrec_b200.ops import sparse_ops as sops
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class PermutePooledEmbeddingsSplit(torch.nn.Module):
    """Reorder the column blocks of a pooled output (differentiable)."""

    def __init__(self, embs_dims: List[int], permute: List[int], device: Optional[torch.device] = None) -> None:
        super().__init__()
        self._dims = list(embs_dims)
        self._permute = list(permute)

    def forward(self, pooled_embs: torch.Tensor) -> torch.Tensor:
        parts = pooled_embs.split(self._dims, dim=1)
        return torch.cat([parts[p] for p in self._permute], dim=1)


class BaseCwEmbeddingSharding(BaseTwEmbeddingSharding[C, F, T, W]):
    _shard_type = ShardingType.COLUMN_WISE

    def __init__(self, sharding_infos: List[EmbeddingShardingInfo], env: ShardingEnv, device: Optional[torch.device] = None,
                 permute_embeddings: bool = False, qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None) -> None:
        super().__init__(sharding_infos, env, device, qcomm_codecs_registry=qcomm_codecs_registry)
        self._permute_embeddings = permute_embeddings
        if self._permute_embeddings:
            self._init_combined_embeddings()

    def _init_combined_embeddings(self) -> None:
        """Several shards of one table may sit on a rank or on different ranks; compute the order that
        puts the shards of each embedding next to each other sorted by column offset."""
        names = super().embedding_names()
        dims = super().embedding_dims()
        metas = super().embedding_shard_metadata()
        by_name: Dict[str, List[Tuple[int, int]]] = {}
        for i, (name, md) in enumerate(zip(names, metas)):
            by_name.setdefault(name, []).append((i, md.shard_offsets[1] if md is not None else 0))
        name_to_index = {n: [i for i, _ in sorted(v, key=lambda t: t[1])] for n, v in by_name.items()}
        combined_names: List[str] = []
        seen: Set[str] = set()
        for n in names:
            if n not in seen:
                combined_names.append(n)
                seen.add(n)
        combined_dims, order = [], []
        for n in combined_names:
            combined_dims.append(sum(dims[i] for i in name_to_index[n]))
            order.extend(name_to_index[n])
        self._embedding_names = names
        self._embedding_dims = dims
        self._embedding_order = order
        self._combined_embedding_names = combined_names
        self._combined_embedding_dims = combined_dims

    def _placements(self, info: EmbeddingShardingInfo):
        """One placement per column block of the table."""
        for rank, shard in zip(info.param_sharding.ranks, info.param_sharding.sharding_spec.shards):
            yield rank, shard, shard.shard_sizes[1]

    def embedding_dims(self) -> List[int]:
        return self._combined_embedding_dims if self._permute_embeddings else self.uncombined_embedding_dims()

    def embedding_names(self) -> List[str]:
        return self._combined_embedding_names if self._permute_embeddings else self.uncombined_embedding_names()

    def uncombined_embedding_dims(self) -> List[int]:
        return super().embedding_dims()

    def uncombined_embedding_names(self) -> List[str]:
        return super().embedding_names()


class CwPooledEmbeddingSharding(_KeySplitPooledRouting, BaseCwEmbeddingSharding[EmbeddingShardingContext, KeyedJaggedTensor, torch.Tensor, torch.Tensor]):
    sharding_type = ShardingType.COLUMN_WISE

    def _output_callbacks(self, device: Optional[torch.device]) -> Optional[List[Callable[[torch.Tensor], torch.Tensor]]]:
        """Put the column blocks of every table next to each other again when they arrive out of order."""
        if not self._permute_embeddings or self._embedding_order == list(range(len(self._embedding_order))):
            return None
        assert len(self._embedding_order) == len(self._embedding_dims)
        return [PermutePooledEmbeddingsSplit(self._embedding_dims, self._embedding_order, device=device)]


_INFER_NAMES = ("InferCwPooledEmbeddingSharding", "InferCwPooledEmbeddingDist", "InferCwPooledEmbeddingDistWithPermute")


def __getattr__(name: str):
    """The inference strategies live in ``infer_shardings`` (they build on every training strategy); they are reachable from
    here under the reference's import path."""
    if name in _INFER_NAMES:
        from torchrec_b200.distributed.sharding import infer_shardings

        return getattr(infer_shardings, name)
    raise AttributeError(name)
