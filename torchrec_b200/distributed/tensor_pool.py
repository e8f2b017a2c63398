"""Sharded ``TensorPool``: the training form (one process per rank, exchanges on the process group) lives in ``object_pool``; this
module adds the inference form, where one process holds every device's row block.
Counterpart of ``torchrec/distributed/tensor_pool.py`` (``ShardedTensorPool`` ``:63``, ``LocalShardPool`` ``:254``,
``ShardedInferenceTensorPool`` ``:300``)."""
from __future__ import annotations

from typing import List, Optional

import torch
from torch import nn

from torchrec_b200.distributed.object_pool import ShardedTensorPool, TensorPoolSharder  # noqa: F401
from torchrec_b200.distributed.types import LazyAwaitable, ObjectPoolShardingPlan, ObjectPoolShardingType, ShardingEnv, rank_device
from torchrec_b200.modules.tensor_pool import TensorPool


class TensorPoolAwaitable(LazyAwaitable[torch.Tensor]):
    """Rows of a lookup whose value exchange may still be in flight."""

    def __init__(self, awaitable, unbucketize_permute: Optional[torch.Tensor] = None) -> None:
        super().__init__()
        self._awaitable, self._permute = awaitable, unbucketize_permute

    def _wait_impl(self) -> torch.Tensor:
        rows = self._awaitable.wait()
        return rows if self._permute is None else rows.index_select(0, self._permute)


def index_select_view(output: torch.Tensor, unbucketize_permute: Optional[torch.Tensor], dim: int) -> torch.Tensor:
    """Rows gathered per block, back in the order of the request: ``output[unbucketize_permute]`` as ``[n, dim]``."""
    return output[unbucketize_permute].view(-1, dim)


def update(shard: torch.nn.Parameter, rank_ids: torch.Tensor, values: torch.Tensor) -> torch.Tensor:
    """Overwrite rows ``rank_ids`` of one device's block with ``values`` (moved to the block's device); returns an empty tensor so
    that the call has a tensor result when it is traced."""
    with torch.no_grad():
        shard.index_copy_(0, rank_ids.to(shard.device).long(), values.to(shard.device, shard.dtype))
    return torch.empty(0)


class LocalShardPool(nn.Module):
    """The row block one device holds: ``forward(local ids) -> rows``; ``update`` overwrites rows in place."""

    def __init__(self, shard: torch.Tensor) -> None:
        super().__init__()
        self._shard = nn.Parameter(shard, requires_grad=False)

    def forward(self, rank_ids: torch.Tensor) -> torch.Tensor:
        return self._shard.index_select(0, rank_ids.to(self._shard.device).long())

    @torch.no_grad()
    def update(self, rank_ids: torch.Tensor, values: torch.Tensor) -> None:
        update(self._shard, rank_ids, values)


class ShardedInferenceTensorPool(nn.Module):
    """A ``TensorPool`` cut into equal row blocks, one per device, all driven by this process: ``lookup(ids)`` splits the ids by block,
    gathers on every device and returns the rows on ``device`` in the order of ``ids``.  Only row-wise plans are served."""

    def __init__(self, env: ShardingEnv, pool_size: int, dim: int, dtype: torch.dtype, plan: ObjectPoolShardingPlan, module: Optional[TensorPool] = None,
                 device: Optional[torch.device] = None) -> None:
        from torchrec_b200.distributed.sharding.rw_tensor_pool_sharding import InferRwTensorPoolSharding

        super().__init__()
        assert plan.sharding_type == ObjectPoolShardingType.ROW_WISE, "an inference tensor pool is sharded row-wise"
        self._pool_size, self._dim, self._dtype = pool_size, dim, dtype
        self._world_size, self._plan = env.world_size, plan
        self._device = device if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self._sharding = InferRwTensorPoolSharding(pool_size, env, self._device)
        kind = self._device.type
        self._devices: List[torch.device] = [rank_device(kind, r) for r in range(self._world_size)]
        sizes = self._sharding.local_pool_size_per_rank
        block = sizes[0]
        shards = []
        for r, (rows, dev) in enumerate(zip(sizes, self._devices)):
            rows = max(rows, 0)
            piece = torch.zeros(rows, dim, dtype=dtype, device=dev)
            if module is not None and module.device.type != "meta" and rows > 0:
                piece.copy_(module.pool[r * block: r * block + rows])
            shards.append(LocalShardPool(piece))
        self._local_shard_pools = nn.ModuleList(shards)
        self._lookup_ids_dist = self._sharding.create_lookup_ids_dist(self._devices)
        self._lookup_values_dist = self._sharding.create_lookup_values_dist()

    @property
    def pool_size(self) -> int:
        return self._pool_size

    @property
    def dim(self) -> int:
        return self._dim

    @property
    def dtype(self) -> torch.dtype:
        return self._dtype

    @property
    def device(self) -> torch.device:
        return self._device

    def lookup(self, ids: torch.Tensor) -> torch.Tensor:
        per_device = self._lookup_ids_dist(ids)
        rows = [pool(local) for pool, local in zip(self._local_shard_pools, per_device)]
        return self._lookup_values_dist(rows, self._lookup_ids_dist.unbucketize_permute)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return self.lookup(ids)

    def update(self, ids: torch.Tensor, values: torch.Tensor) -> None:
        raise NotImplementedError("an inference pool is read-only: load its shards from a trained pool")
