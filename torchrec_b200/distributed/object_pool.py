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


class _RwRouter:
    """Id routing shared by the pools: block size, per-rank counts and the permutation that groups ids by owner."""

    def __init__(self, pool_size: int, env: ShardingEnv) -> None:
        self.world, self.rank, self.pg = env.world_size, env.rank, env.process_group
        self.block = (pool_size + self.world - 1) // self.world
        self.local_rows = max(0, min(self.block, pool_size - self.rank * self.block))

    def route(self, ids: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, List[int], List[int]]:
        """``(order, local ids received here, send counts, receive counts)``; ``ids[order]`` is grouped by owner."""
        ids = ids.long()
        owner = torch.div(ids, self.block, rounding_mode="floor").clamp(max=self.world - 1)
        order = torch.argsort(owner, stable=True)
        send = torch.bincount(owner, minlength=self.world)
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.pg)
        send_l, recv_l = send.tolist(), recv.tolist()
        got = torch.empty(sum(recv_l), dtype=torch.int64, device=ids.device)
        dist.all_to_all_single(got, ids.index_select(0, order).contiguous(), output_split_sizes=recv_l, input_split_sizes=send_l, group=self.pg)
        return order, got - self.rank * self.block, send_l, recv_l

    def exchange(self, payload: torch.Tensor, in_splits: List[int], out_splits: List[int]) -> torch.Tensor:
        out = torch.empty((sum(out_splits),) + tuple(payload.shape[1:]), dtype=payload.dtype, device=payload.device)
        dist.all_to_all_single(out, payload.contiguous(), output_split_sizes=out_splits, input_split_sizes=in_splits, group=self.pg)
        return out


class ShardedTensorPool(nn.Module):
    def __init__(self, module: TensorPool, plan: ObjectPoolShardingPlan, env: ShardingEnv, device: Optional[torch.device] = None) -> None:
        super().__init__()
        self._plan, self._env = plan, env
        self._pool_size, self._dim, self._dtype = module.pool_size, module.dim, module.dtype
        device = device if device is not None else module.device
        if plan.sharding_type == ObjectPoolShardingType.ROW_WISE:
            self._router: Optional[_RwRouter] = _RwRouter(self._pool_size, env)
            rows = self._router.local_rows
            lo = env.rank * self._router.block
        else:
            self._router, rows, lo = None, self._pool_size, 0
        self.register_buffer("_pool", torch.zeros(rows, self._dim, dtype=self._dtype, device=device))
        if module.device.type != "meta" and rows > 0:
            self._pool.copy_(module.pool[lo: lo + rows])

    @property
    def pool_size(self) -> int:
        return self._pool_size

    @property
    def dim(self) -> int:
        return self._dim

    def update(self, ids: torch.Tensor, values: torch.Tensor) -> None:
        ids = ids.to(self._pool.device)
        values = values.to(self._pool.device)
        if self._router is None:
            # replicated: every rank applies every rank's updates
            all_ids = [torch.empty(0)] * self._env.world_size
            gathered_i: List[Optional[torch.Tensor]] = [None] * self._env.world_size
            gathered_v: List[Optional[torch.Tensor]] = [None] * self._env.world_size
            dist.all_gather_object(gathered_i, ids.cpu(), group=self._env.process_group)
            dist.all_gather_object(gathered_v, values.cpu(), group=self._env.process_group)
            for i, v in zip(gathered_i, gathered_v):
                self._pool.index_copy_(0, i.to(self._pool.device).long(), v.to(self._pool.device))
            del all_ids
            return
        order, local_ids, send, recv = self._router.route(ids)
        got = self._router.exchange(values.index_select(0, order), send, recv)
        self._pool.index_copy_(0, local_ids, got)

    def lookup(self, ids: torch.Tensor) -> torch.Tensor:
        ids = ids.to(self._pool.device)
        if self._router is None:
            return self._pool.index_select(0, ids.long())
        order, local_ids, send, recv = self._router.route(ids)
        rows = self._pool.index_select(0, local_ids)
        back = self._router.exchange(rows, recv, send)
        out = torch.empty_like(back)
        out[order] = back
        return out

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return self.lookup(ids)


class ShardedKeyedJaggedTensorPool(nn.Module):
    """Row-wise sharded KJT pool: each rank holds the fixed-capacity rows of its id block; values travel padded."""

    def __init__(self, module: KeyedJaggedTensorPool, plan: ObjectPoolShardingPlan, env: ShardingEnv, device: Optional[torch.device] = None) -> None:
        super().__init__()
        assert plan.sharding_type == ObjectPoolShardingType.ROW_WISE, "KJT pools are row-wise sharded"
        self._router = _RwRouter(module.pool_size, env)
        dev = device if device is not None else module._values.device
        self._local = KeyedJaggedTensorPool(max(self._router.local_rows, 1), module.feature_max_lengths, values_dtype=module._values.dtype, is_weighted=module._is_weighted, device=dev)
        self._keys = list(module.feature_max_lengths.keys())
        self._caps = [module.feature_max_lengths[k] for k in self._keys]
        self._is_weighted = module._is_weighted

    def update(self, ids: torch.Tensor, values: KeyedJaggedTensor) -> None:
        from torchrec_b200.ops import sparse_ops as sops

        dev = self._local._values.device
        ids = ids.to(dev)
        B = ids.numel()
        order, local_ids, send, recv = self._router.route(ids)
        lens = values.lengths().view(len(self._keys), B).t().to(dev)  # [B, F]
        jt = values.to_dict()
        dense = torch.cat([sops.jagged_to_padded_dense(jt[k].values().to(dev), jt[k].offsets().to(dev), cap, 0) if jt[k].values().numel() else
                           torch.zeros(B, cap, dtype=values.values().dtype, device=dev) for k, cap in zip(self._keys, self._caps)], dim=1)
        got_v = self._router.exchange(dense.index_select(0, order), send, recv)
        got_l = self._router.exchange(lens.index_select(0, order), send, recv)
        if local_ids.numel() == 0:
            return
        self._local._values[local_ids] = got_v.to(self._local._values.dtype)
        self._local._lengths[local_ids] = torch.minimum(got_l, torch.tensor(self._caps, device=dev).unsqueeze(0))

    def lookup(self, ids: torch.Tensor) -> KeyedJaggedTensor:
        dev = self._local._values.device
        ids = ids.to(dev)
        B = ids.numel()
        order, local_ids, send, recv = self._router.route(ids)
        rows = self._router.exchange(self._local._values.index_select(0, local_ids), recv, send)
        lens = self._router.exchange(self._local._lengths.index_select(0, local_ids), recv, send)
        v = torch.empty_like(rows)
        l = torch.empty_like(lens)
        v[order], l[order] = rows, lens
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
