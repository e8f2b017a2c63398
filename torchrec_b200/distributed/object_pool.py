"""Sharded object pools: ids are cut into equal row blocks, one block per rank (``ROW_WISE``), or the pool is kept whole on every
rank (``REPLICATED_ROW_WISE``).  ``update`` sends every (id, value) to the rank that owns the id; ``lookup`` sends the ids there and brings
the values back in the caller's order.  Exchanges are plain all-to-alls on the process group (ids first, then payload).
Counterpart of ``torchrec/distributed/tensor_pool.py``, ``keyed_jagged_tensor_pool.py`` and ``sharding/rw_pool_sharding.py``."""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple, Type

import torch
import torch.distributed as dist
from torch import nn

from torchrec_b200.distributed.types import ModuleSharder, ObjectPoolShardingPlan, ObjectPoolShardingType, ShardingEnv
from torchrec_b200.modules.keyed_jagged_tensor_pool import KeyedJaggedTensorPool
from torchrec_b200.modules.tensor_pool import TensorPool
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class ShardedTensorPool(nn.Module):
    """``TensorPool`` whose rows live on their owning rank (row-wise) or on every rank (replicated).  ``update`` / ``lookup`` run
    the id exchange and then the value exchange built by the pool's sharding object."""

    def __init__(self, module: TensorPool, plan: ObjectPoolShardingPlan, env: ShardingEnv, device: Optional[torch.device] = None) -> None:
        from torchrec_b200.distributed.sharding.rw_tensor_pool_sharding import TensorPoolRwReplicatedSharding, TensorPoolRwSharding

        super().__init__()
        self._plan, self._env = plan, env
        self._pool_size, self._dim, self._dtype = module.pool_size, module.dim, module.dtype
        device = device if device is not None else module.device
        self._replicated = plan.sharding_type != ObjectPoolShardingType.ROW_WISE
        cls = TensorPoolRwReplicatedSharding if self._replicated else TensorPoolRwSharding
        self._sharding = cls(self._pool_size, self._dim, env, device)
        rows, lo = self._sharding.local_pool_size, self._sharding.row_offset
        self.register_buffer("_pool", torch.zeros(rows, self._dim, dtype=self._dtype, device=device))
        if module.device.type != "meta" and rows > 0:
            self._pool.copy_(module.pool[lo: lo + rows])
        self._update_ids_dist = self._sharding.create_update_ids_dist()
        self._update_values_dist = self._sharding.create_update_values_dist()
        self._lookup_ids_dist = self._sharding.create_lookup_ids_dist()
        self._lookup_values_dist = self._sharding.create_lookup_values_dist()

    @property
    def pool_size(self) -> int:
        return self._pool_size

    @property
    def dim(self) -> int:
        return self._dim

    def update(self, ids: torch.Tensor, values: torch.Tensor) -> None:
        ctx = self._sharding.create_context()
        local_ids = self._update_ids_dist(ctx, ids.to(self._pool.device))
        rows = self._update_values_dist(ctx, values.to(self._pool.device))
        if local_ids.numel():
            self._pool.index_copy_(0, local_ids, rows.to(self._pool.dtype))

    def lookup(self, ids: torch.Tensor) -> torch.Tensor:
        ids = ids.to(self._pool.device)
        if self._replicated:
            return self._pool.index_select(0, ids.long())
        ctx = self._sharding.create_context()
        local_ids = self._lookup_ids_dist(ctx, ids)
        return self._lookup_values_dist(ctx, self._pool.index_select(0, local_ids))

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return self.lookup(ids)


class ShardedKeyedJaggedTensorPool(nn.Module):
    """Row-wise sharded KJT pool: each rank holds the fixed-capacity rows of its id block; values travel padded."""

    def __init__(self, module: KeyedJaggedTensorPool, plan: ObjectPoolShardingPlan, env: ShardingEnv, device: Optional[torch.device] = None) -> None:
        super().__init__()
        assert plan.sharding_type == ObjectPoolShardingType.ROW_WISE, "KJT pools are row-wise sharded"
        from torchrec_b200.distributed.sharding.rw_kjt_pool_sharding import KeyedJaggedTensorPoolRwSharding

        dev = device if device is not None else module._values.device
        self._sharding = KeyedJaggedTensorPoolRwSharding(module.pool_size, env, dev, num_features=len(module.feature_max_lengths))
        self._update_ids_dist = self._sharding.create_update_ids_dist()
        self._update_values_dist = self._sharding.create_update_values_dist()
        self._lookup_ids_dist = self._sharding.create_lookup_ids_dist()
        self._lookup_values_dist = self._sharding.create_lookup_values_dist()
        self._local = KeyedJaggedTensorPool(max(self._sharding.local_pool_size, 1), module.feature_max_lengths, values_dtype=module._values.dtype, is_weighted=module._is_weighted, device=dev)
        self._keys = list(module.feature_max_lengths.keys())
        self._caps = [module.feature_max_lengths[k] for k in self._keys]
        self._is_weighted = module._is_weighted

    def update(self, ids: torch.Tensor, values: KeyedJaggedTensor) -> None:
        from torchrec_b200.ops import sparse_ops as sops

        dev = self._local._values.device
        ids = ids.to(dev)
        B = ids.numel()
        ctx = self._sharding.create_context()
        local_ids = self._update_ids_dist(ctx, ids)
        lens = values.lengths().view(len(self._keys), B).t().to(dev)  # [B, F]
        jt = values.to_dict()
        dense = torch.cat([sops.jagged_to_padded_dense(jt[k].values().to(dev), jt[k].offsets().to(dev), cap, 0) if jt[k].values().numel() else
                           torch.zeros(B, cap, dtype=values.values().dtype, device=dev) for k, cap in zip(self._keys, self._caps)], dim=1)
        got_v, got_l = self._update_values_dist(ctx, dense, lens)
        if local_ids.numel() == 0:
            return
        self._local._values[local_ids] = got_v.to(self._local._values.dtype)
        self._local._lengths[local_ids] = torch.minimum(got_l, torch.tensor(self._caps, device=dev).unsqueeze(0))

    def lookup(self, ids: torch.Tensor) -> KeyedJaggedTensor:
        dev = self._local._values.device
        ids = ids.to(dev)
        B = ids.numel()
        ctx = self._sharding.create_context()
        local_ids = self._lookup_ids_dist(ctx, ids)
        v, l = self._lookup_values_dist(ctx, self._local._values.index_select(0, local_ids), self._local._lengths.index_select(0, local_ids))
        vals, start = [], 0
        for f, cap in enumerate(self._caps):
            block = v[:, start: start + cap]
            mask = torch.arange(cap, device=dev).unsqueeze(0) < l[:, f: f + 1]
            vals.append(block[mask])
            start += cap
        return KeyedJaggedTensor(keys=self._keys, values=torch.cat(vals), lengths=l.t().reshape(-1), stride=B)

    def forward(self, ids: torch.Tensor) -> KeyedJaggedTensor:
        return self.lookup(ids)


class TensorPoolSharder(ModuleSharder[TensorPool]):
    def shard(self, module: TensorPool, plan: ObjectPoolShardingPlan, env: ShardingEnv, device: Optional[torch.device] = None, module_fqn: Optional[str] = None) -> ShardedTensorPool:
        return ShardedTensorPool(module, plan, env, device)

    @property
    def module_type(self) -> Type[TensorPool]:
        return TensorPool


class KeyedJaggedTensorPoolSharder(ModuleSharder[KeyedJaggedTensorPool]):
    def shard(self, module: KeyedJaggedTensorPool, plan: ObjectPoolShardingPlan, env: ShardingEnv, device: Optional[torch.device] = None,
              module_fqn: Optional[str] = None) -> ShardedKeyedJaggedTensorPool:
        return ShardedKeyedJaggedTensorPool(module, plan, env, device)

    @property
    def module_type(self) -> Type[KeyedJaggedTensorPool]:
        return KeyedJaggedTensorPool
