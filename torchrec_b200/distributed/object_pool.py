"""Sharded object pools: ids are cut into equal row blocks, one block per rank (``ROW_WISE``), or the pool is kept whole on every
rank (``REPLICATED_ROW_WISE``).  ``update`` sends every (id, value) to the rank that owns the id; ``lookup`` sends the ids there and brings
the values back in the caller's order.  Exchanges are plain all-to-alls on the process group (ids first, then payload).
Counterpart of ``torchrec/distributed/tensor_pool.py``, ``keyed_jagged_tensor_pool.py`` and ``sharding/rw_pool_sharding.py``."""
from __future__ import annotations

import abc
from typing import Any, Dict, List, Optional, Tuple, Type

import torch
import torch.distributed as dist
from torch import nn

from torchrec_b200.distributed.types import ModuleSharder, ObjectPoolShardingPlan, ObjectPoolShardingType, ShardingEnv
from torchrec_b200.modules.keyed_jagged_tensor_pool import KeyedJaggedTensorPool
from torchrec_b200.modules.tensor_pool import TensorPool
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class ShardedObjectPool(nn.Module, abc.ABC):
    """The shape every sharded pool has: a distributed key-value store over ids.

    ``update(ids, values)``: check the values, send each id to its owner (``_update_ids_dist``), send the values the same way
    (``_update_values_dist``), write them locally (``_update_local``).  ``lookup(ids)``: send the ids (``_lookup_ids_dist``), read
    locally (``_lookup_local``), bring the values back in the caller's order (``_lookup_values_dist``).  A subclass supplies the
    seven steps.  Counterpart of ``torchrec/distributed/object_pool.py:26-139``."""

    @abc.abstractmethod
    def _create_context(self) -> Any:
        ...

    @abc.abstractmethod
    def _update_preproc(self, values: Any) -> Any:
        """Check and normalise the values of an update."""

    @abc.abstractmethod
    def _update_ids_dist(self, ctx: Any, ids: torch.Tensor) -> torch.Tensor:
        ...

    @abc.abstractmethod
    def _update_values_dist(self, ctx: Any, values: Any) -> Any:
        ...

    @abc.abstractmethod
    def _update_local(self, ctx: Any, ids: torch.Tensor, values: Any) -> None:
        ...

    @abc.abstractmethod
    def _lookup_ids_dist(self, ctx: Any, ids: torch.Tensor) -> torch.Tensor:
        ...

    @abc.abstractmethod
    def _lookup_local(self, ctx: Any, ids: torch.Tensor) -> Any:
        ...

    @abc.abstractmethod
    def _lookup_values_dist(self, ctx: Any, values: Any) -> Any:
        ...

    def update(self, ids: torch.Tensor, values: Any) -> None:
        values = self._update_preproc(values)
        ctx = self._create_context()
        local_ids = self._update_ids_dist(ctx, ids)
        self._update_local(ctx, local_ids, self._update_values_dist(ctx, values))

    def lookup(self, ids: torch.Tensor) -> Any:
        ctx = self._create_context()
        local_ids = self._lookup_ids_dist(ctx, ids)
        return self._lookup_values_dist(ctx, self._lookup_local(ctx, local_ids))

    def forward(self, ids: torch.Tensor) -> Any:
        return self.lookup(ids)


class ShardedTensorPool(ShardedObjectPool):
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
        self._dists = nn.ModuleList([self._sharding.create_update_ids_dist(), self._sharding.create_update_values_dist(),
                                     self._sharding.create_lookup_ids_dist(), self._sharding.create_lookup_values_dist()])

    @property
    def pool_size(self) -> int:
        return self._pool_size

    @property
    def dim(self) -> int:
        return self._dim

    def _create_context(self):
        return self._sharding.create_context()

    def _update_preproc(self, values: torch.Tensor) -> torch.Tensor:
        assert values.dim() == 2 and values.shape[1] == self._dim, f"values must be [n, {self._dim}], got {tuple(values.shape)}"
        return values.to(self._pool.device)

    def _update_ids_dist(self, ctx, ids: torch.Tensor) -> torch.Tensor:
        return self._dists[0](ctx, ids.to(self._pool.device))

    def _update_values_dist(self, ctx, values: torch.Tensor) -> torch.Tensor:
        return self._dists[1](ctx, values)

    def _update_local(self, ctx, ids: torch.Tensor, values: torch.Tensor) -> None:
        if ids.numel():
            self._pool.index_copy_(0, ids, values.to(self._pool.dtype))

    def _lookup_ids_dist(self, ctx, ids: torch.Tensor) -> torch.Tensor:
        return self._dists[2](ctx, ids.to(self._pool.device))

    def _lookup_local(self, ctx, ids: torch.Tensor) -> torch.Tensor:
        return self._pool.index_select(0, ids)

    def _lookup_values_dist(self, ctx, values: torch.Tensor) -> torch.Tensor:
        return self._dists[3](ctx, values)

    def lookup(self, ids: torch.Tensor) -> torch.Tensor:
        if self._replicated:  # every rank holds every row: no exchange
            return self._pool.index_select(0, ids.to(self._pool.device).long())
        return super().lookup(ids)


class ShardedKeyedJaggedTensorPool(ShardedObjectPool):
    """Row-wise sharded KJT pool: each rank holds the fixed-capacity rows of its id block; values travel padded."""

    def __init__(self, module: KeyedJaggedTensorPool, plan: ObjectPoolShardingPlan, env: ShardingEnv, device: Optional[torch.device] = None) -> None:
        super().__init__()
        assert plan.sharding_type == ObjectPoolShardingType.ROW_WISE, "KJT pools are row-wise sharded"
        from torchrec_b200.distributed.sharding.rw_kjt_pool_sharding import KeyedJaggedTensorPoolRwSharding

        dev = device if device is not None else module._values.device
        self._sharding = KeyedJaggedTensorPoolRwSharding(module.pool_size, env, dev, num_features=len(module.feature_max_lengths))
        self._dists = nn.ModuleList([self._sharding.create_update_ids_dist(), self._sharding.create_update_values_dist(),
                                     self._sharding.create_lookup_ids_dist(), self._sharding.create_lookup_values_dist()])
        self._local = KeyedJaggedTensorPool(max(self._sharding.local_pool_size, 1), module.feature_max_lengths, values_dtype=module._values.dtype, is_weighted=module._is_weighted, device=dev)
        self._keys = list(module.feature_max_lengths.keys())
        self._caps = [module.feature_max_lengths[k] for k in self._keys]
        self._is_weighted = module._is_weighted

    def _create_context(self):
        return self._sharding.create_context()

    def _update_preproc(self, values: KeyedJaggedTensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """The KJT as what travels: every feature padded to its capacity, ``[B, sum(caps)]``, and the lengths ``[B, F]``."""
        from torchrec_b200.ops import sparse_ops as sops

        assert values.keys() == self._keys, f"the pool holds {self._keys}, the update has {values.keys()}"
        dev = self._local._values.device
        B = values.stride()
        lens = values.lengths().view(len(self._keys), B).t().to(dev)
        jt = values.to_dict()
        dense = torch.cat([sops.jagged_to_padded_dense(jt[k].values().to(dev), jt[k].offsets().to(dev), cap, 0) if jt[k].values().numel() else
                           torch.zeros(B, cap, dtype=values.values().dtype, device=dev) for k, cap in zip(self._keys, self._caps)], dim=1)
        return dense, lens

    def _update_ids_dist(self, ctx, ids: torch.Tensor) -> torch.Tensor:
        return self._dists[0](ctx, ids.to(self._local._values.device))

    def _update_values_dist(self, ctx, values: Tuple[torch.Tensor, torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
        return self._dists[1](ctx, values[0], values[1])

    def _update_local(self, ctx, ids: torch.Tensor, values: Tuple[torch.Tensor, torch.Tensor]) -> None:
        if ids.numel() == 0:
            return
        got_v, got_l = values
        self._local._values[ids] = got_v.to(self._local._values.dtype)
        self._local._lengths[ids] = torch.minimum(got_l, torch.tensor(self._caps, device=got_l.device).unsqueeze(0))

    def _lookup_ids_dist(self, ctx, ids: torch.Tensor) -> torch.Tensor:
        return self._dists[2](ctx, ids.to(self._local._values.device))

    def _lookup_local(self, ctx, ids: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        return self._local._values.index_select(0, ids), self._local._lengths.index_select(0, ids)

    def _lookup_values_dist(self, ctx, values: Tuple[torch.Tensor, torch.Tensor]) -> KeyedJaggedTensor:
        v, l = self._dists[3](ctx, values[0], values[1])
        dev = v.device
        vals, start = [], 0
        for f, cap in enumerate(self._caps):
            block = v[:, start: start + cap]
            mask = torch.arange(cap, device=dev).unsqueeze(0) < l[:, f: f + 1]
            vals.append(block[mask])
            start += cap
        return KeyedJaggedTensor(keys=self._keys, values=torch.cat(vals), lengths=l.t().reshape(-1), stride=v.shape[0])


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
