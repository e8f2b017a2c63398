"""Value exchange of row-wise sharded tensor pools: ``[n, dim]`` rows follow the ids of the preceding id exchange.

Update: rows are grouped like the ids and sent to the owners.  Lookup: owners send the selected rows back along the reverse
splits and the caller's order is restored.  Counterpart of ``torchrec/distributed/sharding/rw_tensor_pool_sharding.py:40-270``."""
from __future__ import annotations

from typing import Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import nn

from torchrec_b200.distributed.sharding.rw_pool_sharding import InferRwObjectPoolSharding, ObjectPoolReplicatedRwSharding, ObjectPoolRwSharding
from torchrec_b200.distributed.tensor_sharding import ObjectPoolRwShardingContext, TensorPoolRwShardingContext
from torchrec_b200.distributed.types import ShardingEnv


def exchange_rows(pg: dist.ProcessGroup, payload: torch.Tensor, in_splits: List[int], out_splits: List[int]) -> torch.Tensor:
    """All-to-all of whole rows (dim 0) with the given per-rank row counts."""
    out = torch.empty((sum(out_splits),) + tuple(payload.shape[1:]), dtype=payload.dtype, device=payload.device)
    dist.all_to_all_single(out, payload.contiguous(), output_split_sizes=out_splits, input_split_sizes=in_splits, group=pg)
    return out


class RwTensorPoolValuesDist(nn.Module):
    def __init__(self, pg: dist.ProcessGroup, is_update: bool) -> None:
        super().__init__()
        self._pg, self._is_update = pg, is_update

    def forward(self, ctx: ObjectPoolRwShardingContext, values: torch.Tensor) -> torch.Tensor:
        if self._is_update:
            return exchange_rows(self._pg, values.index_select(0, ctx.bucketize_permute), ctx.send_splits, ctx.receive_splits)
        back = exchange_rows(self._pg, values, ctx.receive_splits, ctx.send_splits)
        return back.index_select(0, ctx.unbucketize_permute)


class RwTensorPoolReplicatedValuesDist(nn.Module):
    """Update path of a replicated pool: all-gather the rows (padded to the longest contribution)."""

    def __init__(self, pg: dist.ProcessGroup, world_size: int) -> None:
        super().__init__()
        self._pg, self._world = pg, world_size

    def forward(self, ctx: ObjectPoolRwShardingContext, values: torch.Tensor) -> torch.Tensor:
        longest = max(ctx.receive_splits) if ctx.receive_splits else 0
        padded = torch.zeros((longest,) + tuple(values.shape[1:]), dtype=values.dtype, device=values.device)
        padded[: values.shape[0]] = values
        bufs = [torch.empty_like(padded) for _ in range(self._world)]
        dist.all_gather(bufs, padded, group=self._pg)
        return torch.cat([b[:n] for b, n in zip(bufs, ctx.receive_splits)])


class TensorPoolRwSharding(ObjectPoolRwSharding):
    def __init__(self, pool_size: int, dim: int, env: ShardingEnv, device: torch.device) -> None:
        super().__init__(pool_size, env, device)
        self._dim = dim

    def create_update_values_dist(self) -> RwTensorPoolValuesDist:
        return RwTensorPoolValuesDist(self._pg, is_update=True)

    def create_lookup_values_dist(self) -> RwTensorPoolValuesDist:
        return RwTensorPoolValuesDist(self._pg, is_update=False)

    def get_sharded_states_to_register(self, pool: Optional[torch.Tensor] = None) -> Iterable[Tuple[str, torch.Tensor]]:
        if pool is not None:
            yield "_pool", pool

    def create_context(self) -> TensorPoolRwShardingContext:
        return TensorPoolRwShardingContext(block_size=torch.tensor([self._block_size], device=self._device))


class TensorPoolRwReplicatedSharding(ObjectPoolReplicatedRwSharding):
    def __init__(self, pool_size: int, dim: int, env: ShardingEnv, device: torch.device) -> None:
        super().__init__(pool_size, env, device)
        self._dim = dim

    def create_update_values_dist(self) -> RwTensorPoolReplicatedValuesDist:
        return RwTensorPoolReplicatedValuesDist(self._pg, self._world_size)

    def create_lookup_values_dist(self) -> nn.Module:
        return nn.Identity()

    def get_sharded_states_to_register(self, pool: Optional[torch.Tensor] = None) -> Iterable[Tuple[str, torch.Tensor]]:
        if pool is not None:
            yield "_pool", pool


class InferRwTensorPoolOutputDist(nn.Module):
    """Bring the per-device rows to one device and restore the caller's order."""

    def __init__(self, device: torch.device) -> None:
        super().__init__()
        self._device = device

    def forward(self, rows_per_device: List[torch.Tensor], unbucketize_permute: torch.Tensor) -> torch.Tensor:
        merged = torch.cat([r.to(self._device, non_blocking=True) for r in rows_per_device])
        return merged.index_select(0, unbucketize_permute.to(self._device))


class InferRwTensorPoolSharding(InferRwObjectPoolSharding):
    def create_lookup_values_dist(self) -> InferRwTensorPoolOutputDist:
        return InferRwTensorPoolOutputDist(self._device)
