"""Contexts and interfaces of sharded object pools (tensor pools, KJT pools).

A pool is sharded by id: rank ``r`` owns ids ``[r * block, (r + 1) * block)``.  One ``update`` or ``lookup`` call carries a context
from the id exchange to the value exchange: the caller's ids, the permutation that groups them by owner (and its inverse), and
how many ids travel between every pair of ranks.  Counterpart of ``torchrec/distributed/tensor_sharding.py:22-134``."""
from __future__ import annotations

import abc
from dataclasses import dataclass, field
from typing import Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist

from torchrec_b200.distributed.types import ShardingEnv
from torchrec_b200.streamable import Multistreamable


def _record(stream: torch.Stream, *tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and t.is_cuda:
            t.record_stream(stream)


@dataclass
class ObjectPoolShardingContext(Multistreamable):
    ids_before_input_dist: Optional[torch.Tensor] = None
    num_ids_each_rank_to_receive: Optional[torch.Tensor] = None
    num_ids_each_rank_to_send: Optional[torch.Tensor] = None
    bucketize_permute: Optional[torch.Tensor] = None
    unbucketize_permute: Optional[torch.Tensor] = None
    # host copies of the two count vectors: the value exchange needs them as split sizes
    send_splits: List[int] = field(default_factory=list)
    receive_splits: List[int] = field(default_factory=list)

    def record_stream(self, stream: torch.Stream) -> None:
        _record(stream, self.ids_before_input_dist, self.num_ids_each_rank_to_receive, self.num_ids_each_rank_to_send,
                self.bucketize_permute, self.unbucketize_permute)


@dataclass
class RwShardingContext(Multistreamable):
    block_size: Optional[torch.Tensor] = None

    def record_stream(self, stream: torch.Stream) -> None:
        _record(stream, self.block_size)


@dataclass
class ObjectPoolRwShardingContext(ObjectPoolShardingContext, RwShardingContext):
    def record_stream(self, stream: torch.Stream) -> None:
        ObjectPoolShardingContext.record_stream(self, stream)
        RwShardingContext.record_stream(self, stream)


@dataclass
class ObjectPoolReplicatedRwShardingContext(ObjectPoolRwShardingContext):
    pass


@dataclass
class TensorPoolRwShardingContext(ObjectPoolRwShardingContext):
    pass


class ObjectPoolSharding(abc.ABC):
    """Factory of the four exchanges of a sharded pool and of its local state."""

    @abc.abstractmethod
    def create_update_ids_dist(self) -> torch.nn.Module: ...

    @abc.abstractmethod
    def create_update_values_dist(self) -> torch.nn.Module: ...

    @abc.abstractmethod
    def create_lookup_ids_dist(self) -> torch.nn.Module: ...

    @abc.abstractmethod
    def create_lookup_values_dist(self) -> torch.nn.Module: ...

    @abc.abstractmethod
    def get_sharded_states_to_register(self) -> Iterable[Tuple[str, torch.Tensor]]: ...

    @abc.abstractmethod
    def create_context(self) -> ObjectPoolShardingContext: ...


class InferObjectPoolSharding(abc.ABC):
    """Single-process, one-shard-per-device pool sharding for inference: equal row blocks, the last one holds the remainder."""

    def __init__(self, pool_size: int, env: ShardingEnv, device: torch.device) -> None:
        self._pool_size = pool_size
        self._env = env
        self._pg: Optional[dist.ProcessGroup] = env.process_group
        self._world_size: int = env.world_size
        self._rank: int = env.rank
        self._device = device
        self._block_size: int = (pool_size + self._world_size - 1) // self._world_size
        self._last_block_size: int = pool_size - self._block_size * (self._world_size - 1)
        self.local_pool_size_per_rank: List[int] = [self._block_size] * (self._world_size - 1) + [self._last_block_size]
        self._block_size_t: torch.Tensor = torch.tensor([self._block_size], device=device, dtype=torch.long)

    @abc.abstractmethod
    def create_lookup_ids_dist(self) -> torch.nn.Module: ...

    @abc.abstractmethod
    def create_lookup_values_dist(self) -> torch.nn.Module: ...
