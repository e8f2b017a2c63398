"""Sharded ``KeyedJaggedTensorPool``: the training form lives in ``object_pool``; this module adds the inference form, where one
process holds every device's block of pool rows.  Counterpart of ``torchrec/distributed/keyed_jagged_tensor_pool.py``
(``ShardedKeyedJaggedTensorPool`` ``:135``, ``ShardedInferenceKeyedJaggedTensorPool`` ``:490``)."""
from __future__ import annotations

from typing import List, Optional

import torch
from torch import nn

from torchrec_b200.distributed.object_pool import KeyedJaggedTensorPoolSharder, ShardedKeyedJaggedTensorPool  # noqa: F401
from torchrec_b200.distributed.types import LazyAwaitable, ObjectPoolShardingPlan, ObjectPoolShardingType, ShardingEnv, rank_device
from torchrec_b200.modules.keyed_jagged_tensor_pool import KeyedJaggedTensorPool
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class KeyedJaggedTensorPoolAwaitable(LazyAwaitable[KeyedJaggedTensor]):
    """A pool lookup whose padded rows may still be in flight; waiting packs them into a KJT."""

    def __init__(self, awaitable, keys: List[str], caps: List[int], batch: int) -> None:
        super().__init__()
        self._awaitable, self._keys, self._caps, self._batch = awaitable, keys, caps, batch

    def _wait_impl(self) -> KeyedJaggedTensor:
        values, lengths = self._awaitable.wait()
        return _pack(values, lengths, self._keys, self._caps, self._batch)


def _pack(values: torch.Tensor, lengths: torch.Tensor, keys: List[str], caps: List[int], batch: int) -> KeyedJaggedTensor:
    """Padded rows ``[B, sum(caps)]`` and lengths ``[B, F]`` -> feature-major KJT."""
    parts, start = [], 0
    for f, cap in enumerate(caps):
        block = values[:, start: start + cap]
        parts.append(block[torch.arange(cap, device=values.device).unsqueeze(0) < lengths[:, f: f + 1]])
        start += cap
    return KeyedJaggedTensor(keys=keys, values=torch.cat(parts) if parts else values.new_zeros(0), lengths=lengths.t().reshape(-1), stride=batch)


class ShardedInferenceKeyedJaggedTensorPool(nn.Module):
    """A KJT pool cut into equal row blocks, one per device, all driven by this process: ``lookup(ids)`` splits the ids by block, reads
    the padded rows and lengths on every device, merges them on ``device`` in the order of ``ids`` and packs the KJT."""

    def __init__(self, env: ShardingEnv, pool_size: int, feature_max_lengths, values_dtype: torch.dtype, is_weighted: bool, plan: ObjectPoolShardingPlan,
                 module: Optional[KeyedJaggedTensorPool] = None, device: Optional[torch.device] = None) -> None:
        from torchrec_b200.distributed.sharding.rw_kjt_pool_sharding import InferRwKeyedJaggedTensorPoolSharding

        super().__init__()
        assert plan.sharding_type == ObjectPoolShardingType.ROW_WISE, "an inference KJT pool is sharded row-wise"
        assert not is_weighted, "weighted KJT pools are not served by the inference form"
        self._pool_size, self._world_size = pool_size, env.world_size
        self._keys = list(feature_max_lengths.keys())
        self._caps = [feature_max_lengths[k] for k in self._keys]
        self._device = device if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self._sharding = InferRwKeyedJaggedTensorPoolSharding(pool_size, env, self._device)
        self._devices = [rank_device(self._device.type, r) for r in range(self._world_size)]
        sizes = self._sharding.local_pool_size_per_rank
        block = sizes[0]
        self._local_pools = nn.ModuleList()
        for r, (rows, dev) in enumerate(zip(sizes, self._devices)):
            local = KeyedJaggedTensorPool(max(rows, 1), dict(feature_max_lengths), values_dtype=values_dtype, is_weighted=False, device=dev)
            if module is not None and module._values.device.type != "meta" and rows > 0:
                local._values[:rows].copy_(module._values[r * block: r * block + rows])
                local._lengths[:rows].copy_(module._lengths[r * block: r * block + rows])
            self._local_pools.append(local)
        self._lookup_ids_dist = self._sharding.create_lookup_ids_dist(self._devices)
        self._lookup_values_dist = self._sharding.create_lookup_values_dist()

    @property
    def pool_size(self) -> int:
        return self._pool_size

    def lookup(self, ids: torch.Tensor) -> KeyedJaggedTensor:
        per_device = self._lookup_ids_dist(ids)
        rows = [pool._values.index_select(0, local.long()) for pool, local in zip(self._local_pools, per_device)]
        lens = [pool._lengths.index_select(0, local.long()) for pool, local in zip(self._local_pools, per_device)]
        values, lengths = self._lookup_values_dist(rows, lens, self._lookup_ids_dist.unbucketize_permute)
        return _pack(values, lengths, self._keys, self._caps, ids.numel())

    def forward(self, ids: torch.Tensor) -> KeyedJaggedTensor:
        return self.lookup(ids)

    def update(self, ids: torch.Tensor, values: KeyedJaggedTensor) -> None:
        raise NotImplementedError("an inference pool is read-only: load its shards from a trained pool")
