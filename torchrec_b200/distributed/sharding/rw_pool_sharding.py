"""Id exchange of row-wise sharded object pools.

``RwObjectPoolIDsDist`` groups the caller's ids by owning rank (stable, so equal ids keep their order and the last update wins),
exchanges the counts and then the ids, and returns this rank's *local* ids; the permutation and the counts stay in the context
for the value exchange that follows.  The replicated variant all-gathers update ids so every rank applies every update, and
answers lookups locally.  Counterpart of ``torchrec/distributed/sharding/rw_pool_sharding.py:60-297``."""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist
from torch import nn

from torchrec_b200.distributed.tensor_sharding import (
    InferObjectPoolSharding,
    ObjectPoolReplicatedRwShardingContext,
    ObjectPoolRwShardingContext,
    ObjectPoolSharding,
)
from torchrec_b200.distributed.types import ShardingEnv


class RwObjectPoolIDsDist(nn.Module):
    def __init__(self, pg: dist.ProcessGroup, world_size: int, rank: int, block_size: int) -> None:
        super().__init__()
        self._pg, self._world, self._rank, self._block = pg, world_size, rank, block_size

    def forward(self, ctx: ObjectPoolRwShardingContext, ids: torch.Tensor) -> torch.Tensor:
        ids = ids.long()
        owner = torch.div(ids, self._block, rounding_mode="floor").clamp(max=self._world - 1)
        order = torch.argsort(owner, stable=True)
        send = torch.bincount(owner, minlength=self._world)
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self._pg)
        ctx.ids_before_input_dist = ids
        ctx.bucketize_permute = order
        ctx.unbucketize_permute = torch.empty_like(order).scatter_(0, order, torch.arange(order.numel(), device=order.device))
        ctx.num_ids_each_rank_to_send, ctx.num_ids_each_rank_to_receive = send, recv
        ctx.send_splits, ctx.receive_splits = send.tolist(), recv.tolist()
        ctx.block_size = torch.tensor([self._block], device=ids.device)
        got = torch.empty(sum(ctx.receive_splits), dtype=torch.int64, device=ids.device)
        dist.all_to_all_single(got, ids.index_select(0, order).contiguous(), output_split_sizes=ctx.receive_splits, input_split_sizes=ctx.send_splits, group=self._pg)
        return got - self._rank * self._block


class RwObjectPoolReplicatedIDsDist(nn.Module):
    """Update path of a replicated pool: every rank receives every rank's ids (global ids: each rank holds the whole pool)."""

    def __init__(self, pg: dist.ProcessGroup, world_size: int) -> None:
        super().__init__()
        self._pg, self._world = pg, world_size

    def forward(self, ctx: ObjectPoolReplicatedRwShardingContext, ids: torch.Tensor) -> torch.Tensor:
        ids = ids.long()
        counts = [torch.zeros(1, dtype=torch.int64, device=ids.device) for _ in range(self._world)]
        dist.all_gather(counts, torch.tensor([ids.numel()], dtype=torch.int64, device=ids.device), group=self._pg)
        ctx.receive_splits = [int(c) for c in counts]
        ctx.send_splits = [ids.numel()] * self._world
        ctx.ids_before_input_dist = ids
        parts = [torch.empty(n, dtype=torch.int64, device=ids.device) for n in ctx.receive_splits]
        dist.all_gather(parts, ids.contiguous(), group=self._pg) if len(set(ctx.receive_splits)) == 1 else self._uneven_gather(parts, ids)
        return torch.cat(parts)

    def _uneven_gather(self, parts: List[torch.Tensor], ids: torch.Tensor) -> None:
        # all_gather needs equal sizes: pad to the longest, trim on arrival
        longest = max(p.numel() for p in parts)
        padded = torch.zeros(longest, dtype=ids.dtype, device=ids.device)
        padded[: ids.numel()] = ids
        bufs = [torch.empty(longest, dtype=ids.dtype, device=ids.device) for _ in parts]
        dist.all_gather(bufs, padded, group=self._pg)
        for p, b in zip(parts, bufs):
            p.copy_(b[: p.numel()])


class ObjectPoolRwSharding(ObjectPoolSharding):
    def __init__(self, pool_size: int, env: ShardingEnv, device: torch.device) -> None:
        self._pool_size, self._env, self._device = pool_size, env, device
        self._pg, self._world_size, self._rank = env.process_group, env.world_size, env.rank
        self._block_size = (pool_size + self._world_size - 1) // self._world_size
        self.local_pool_size = max(0, min(self._block_size, pool_size - self._rank * self._block_size))
        self.row_offset = self._rank * self._block_size

    def create_update_ids_dist(self) -> RwObjectPoolIDsDist:
        return RwObjectPoolIDsDist(self._pg, self._world_size, self._rank, self._block_size)

    def create_lookup_ids_dist(self) -> RwObjectPoolIDsDist:
        return RwObjectPoolIDsDist(self._pg, self._world_size, self._rank, self._block_size)

    def create_context(self) -> ObjectPoolRwShardingContext:
        return ObjectPoolRwShardingContext(block_size=torch.tensor([self._block_size], device=self._device))


class ObjectPoolReplicatedRwSharding(ObjectPoolRwSharding):
    """Every rank keeps the whole pool: updates are broadcast, lookups are local."""

    def __init__(self, pool_size: int, env: ShardingEnv, device: torch.device) -> None:
        super().__init__(pool_size, env, device)
        self.local_pool_size, self.row_offset = pool_size, 0

    def create_update_ids_dist(self) -> RwObjectPoolReplicatedIDsDist:  # type: ignore[override]
        return RwObjectPoolReplicatedIDsDist(self._pg, self._world_size)

    def create_context(self) -> ObjectPoolReplicatedRwShardingContext:
        return ObjectPoolReplicatedRwShardingContext(block_size=torch.tensor([self._block_size], device=self._device))


class InferRwObjectPoolInputDist(nn.Module):
    """Single process, one shard per device: split the ids by row block and move each part to its device (local ids)."""

    def __init__(self, world_size: int, block_size: int, devices: Optional[List[torch.device]] = None) -> None:
        super().__init__()
        self._world, self._block, self._devices = world_size, block_size, devices
        self.unbucketize_permute: Optional[torch.Tensor] = None

    def forward(self, ids: torch.Tensor) -> List[torch.Tensor]:
        ids = ids.long()
        owner = torch.div(ids, self._block, rounding_mode="floor").clamp(max=self._world - 1)
        order = torch.argsort(owner, stable=True)
        self.unbucketize_permute = torch.empty_like(order).scatter_(0, order, torch.arange(order.numel(), device=order.device))
        parts = torch.split(ids.index_select(0, order), torch.bincount(owner, minlength=self._world).tolist())
        out = [p - r * self._block for r, p in enumerate(parts)]
        return [p.to(d, non_blocking=True) for p, d in zip(out, self._devices)] if self._devices else out


class InferRwObjectPoolSharding(InferObjectPoolSharding):
    def create_lookup_ids_dist(self, devices: Optional[List[torch.device]] = None) -> InferRwObjectPoolInputDist:
        return InferRwObjectPoolInputDist(self._world_size, self._block_size, devices)

    def create_lookup_values_dist(self) -> nn.Module:
        raise NotImplementedError("value merge is defined by the pool type (tensor pool, KJT pool)")
