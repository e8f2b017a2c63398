"""Small helpers of the planner (cf. ``torchrec/distributed/planner/utils.py``)."""
from __future__ import annotations

import math
import operator
from functools import reduce
from typing import Any, Callable, Iterable, List, Optional, Type, Union

import torch

from torchrec_b200.distributed.planner.types import Perf, ShardingOption, Storage


def sharder_name(t: Type[Any]) -> str:
    return t.__module__ + "." + t.__name__


def bytes_to_gb(num_bytes: int) -> float:
    return float(num_bytes / (1024 * 1024 * 1024))


def bytes_to_mb(num_bytes: Union[float, int]) -> float:
    return float(num_bytes / (1024 * 1024))


def gb_to_bytes(gb: float) -> int:
    return int(gb * 1024 * 1024 * 1024)


def prod(iterable: Iterable[int]) -> int:
    return reduce(operator.mul, iterable, 1)


def placement(compute_device: str, rank: int, local_size: int) -> str:
    param_device = compute_device
    if compute_device in {"cuda", "mtia"}:
        param_device = f"{compute_device}:{rank % local_size}"
    return f"rank:{rank}/{param_device}"


def storage_repr_in_gb(storage: Optional[Storage]) -> str:
    if storage is None:
        return ""
    return f"Storage(hbm = {round(bytes_to_gb(storage.hbm), 3)} GB, ddr = {round(bytes_to_gb(storage.ddr), 3)} GB)"


def reset_shard_rank(proposal: List[ShardingOption]) -> None:
    for so in proposal:
        for shard in so.shards:
            shard.rank = None


def _find_imbalance_tables(sharding_options: List[ShardingOption], target_imbalance: str = "perf") -> List[ShardingOption]:
    """Options that have a shard on the most loaded rank."""
    rank_to_value = {}
    for so in sharding_options:
        for shard in so.shards:
            v = shard.perf.total if target_imbalance == "perf" else shard.storage.hbm
            rank_to_value[shard.rank] = rank_to_value.get(shard.rank, 0) + v
    if not rank_to_value:
        return []
    max_rank = max(rank_to_value, key=lambda r: rank_to_value[r])
    return [so for so in sharding_options if any(s.rank == max_rank for s in so.shards)]


class BinarySearchPredicate:
    """Binary search over an integer range driven by external feedback (used to size caches)."""

    def __init__(self, A: int, B: int, tolerance: int) -> None:
        self.left, self.right, self.tolerance = A, B, tolerance
        self.first = True

    def next(self, prior_result: bool) -> Optional[int]:
        if self.right - self.left < self.tolerance:
            return None
        mid = self._mid()
        if self.first:
            self.first = False
            return mid
        if prior_result:
            self.left = mid + 1
        else:
            self.right = mid - 1
        if self.right - self.left < self.tolerance:
            return None
        return self._mid()

    def _mid(self) -> int:
        return self.left + ((self.right - self.left) // 2)
