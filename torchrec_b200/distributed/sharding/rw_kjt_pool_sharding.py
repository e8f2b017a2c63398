"""Value exchange of row-wise sharded KJT pools.  A pool row is one sample of every feature with a fixed capacity per feature, so
rows travel as a padded ``[n, sum(capacity)]`` block together with their ``[n, F]`` lengths: two row exchanges along the splits of
the preceding id exchange.  Counterpart of ``torchrec/distributed/sharding/rw_kjt_pool_sharding.py:40-543``."""
from __future__ import annotations

from typing import Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import nn

from torchrec_b200.distributed.sharding.rw_pool_sharding import InferRwObjectPoolSharding, ObjectPoolRwSharding
from torchrec_b200.distributed.sharding.rw_tensor_pool_sharding import RwTensorPoolValuesDist
from torchrec_b200.distributed.tensor_sharding import ObjectPoolRwShardingContext
from torchrec_b200.distributed.types import ShardingEnv


class RwKeyedJaggedTensorPoolUpdateValuesDist(nn.Module):
    def __init__(self, pg: dist.ProcessGroup) -> None:
        super().__init__()
        self._rows = RwTensorPoolValuesDist(pg, is_update=True)

    def forward(self, ctx: ObjectPoolRwShardingContext, padded_values: torch.Tensor, lengths: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        return self._rows(ctx, padded_values), self._rows(ctx, lengths)


class RwKeyedJaggedTensorPoolLookupValuesDist(nn.Module):
    def __init__(self, pg: dist.ProcessGroup) -> None:
        super().__init__()
        self._rows = RwTensorPoolValuesDist(pg, is_update=False)

    def forward(self, ctx: ObjectPoolRwShardingContext, padded_values: torch.Tensor, lengths: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        return self._rows(ctx, padded_values), self._rows(ctx, lengths)


class KeyedJaggedTensorPoolRwSharding(ObjectPoolRwSharding):
    def __init__(self, pool_size: int, env: ShardingEnv, device: torch.device, num_features: int = 0) -> None:
        super().__init__(pool_size, env, device)
        self._num_features = num_features

    def create_update_values_dist(self) -> RwKeyedJaggedTensorPoolUpdateValuesDist:
        return RwKeyedJaggedTensorPoolUpdateValuesDist(self._pg)

    def create_lookup_values_dist(self) -> RwKeyedJaggedTensorPoolLookupValuesDist:
        return RwKeyedJaggedTensorPoolLookupValuesDist(self._pg)

    def get_sharded_states_to_register(self, values: Optional[torch.Tensor] = None, lengths: Optional[torch.Tensor] = None) -> Iterable[Tuple[str, torch.Tensor]]:
        if values is not None:
            yield "values", values
        if lengths is not None:
            yield "key_lengths", lengths


class InferRwKeyedJaggedTensorPoolOutputDist(nn.Module):
    """Merge the per-device padded rows and lengths on one device in the caller's order."""

    def __init__(self, device: torch.device) -> None:
        super().__init__()
        self._device = device

    def forward(self, rows: List[torch.Tensor], lengths: List[torch.Tensor], unbucketize_permute: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        perm = unbucketize_permute.to(self._device)
        v = torch.cat([r.to(self._device, non_blocking=True) for r in rows]).index_select(0, perm)
        l = torch.cat([x.to(self._device, non_blocking=True) for x in lengths]).index_select(0, perm)
        return v, l


class InferRwKeyedJaggedTensorPoolSharding(InferRwObjectPoolSharding):
    def create_lookup_values_dist(self) -> InferRwKeyedJaggedTensorPoolOutputDist:
        return InferRwKeyedJaggedTensorPoolOutputDist(self._device)
