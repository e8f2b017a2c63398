"""Small helpers of the planner (cf. ``torchrec/distributed/planner/utils.py``)."""
from __future__ import annotations

import math
import operator
from functools import reduce
from typing import Any, Callable, Iterable, List, Optional, Tuple, Type, Union

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


def mb_to_bytes(mb: float) -> int:
    return int(mb * 1024 * 1024)


class LuusJaakolaSearch:
    """Derivative-free minimisation of a scalar function on ``[A, B]`` by a clamped Luus-Jaakola random search: keep the best point
    ``x``; probe ``y = clamp(x + u)`` with ``u`` uniform in ``[-d, d]``; a probe that is at least as good becomes the new ``x``, and the
    step ``d`` shrinks by 5 % whenever that happens.  Probes never leave the interval, and a boundary whose cost is already
    known is not probed again.

    Protocol: ``y = s.next(0.0)`` gives the first point; every further ``s.next(f(y))`` reports the cost of the previous point and
    returns the next one, or ``None`` after ``max_iterations`` costs; ``s.best()`` is the best ``(x, f(x))`` seen.
    (``torchrec/distributed/planner/utils.py:177-265`` of the reference.)"""

    def __init__(self, A: float, B: float, max_iterations: int, seed: int = 42, left_cost: Optional[float] = None) -> None:
        import torch

        self.left, self.right = float(A), float(B)
        self.max_iterations = max_iterations
        self.iteration = -1
        self.gen = torch.Generator().manual_seed(seed)
        self.d = self.right - self.left
        self.x = self.uniform(self.left, self.right)
        self.fx = 0.0
        self.y = float("nan")
        self.fleft: Optional[float] = left_cost
        self.fright: Optional[float] = None

    def uniform(self, A: float, B: float) -> float:
        import torch

        return A + (B - A) * float(torch.rand(1, generator=self.gen).item())

    def clamp(self, x: float) -> float:
        return min(max(x, self.left), self.right)

    def shrink_right(self, B: float) -> None:
        """The caller learned that everything from ``B`` on is infeasible: pull the right end in and treat its cost as infinite."""
        self.right = float(B)
        self.fright = float("inf")
        self.d = self.right - self.left
        self.x = self.clamp(self.x)

    def next(self, fy: float) -> Optional[float]:
        self.iteration += 1
        if self.iteration == 0:
            return self.x  # the starting point itself is the first probe
        if self.iteration == 1:
            self.fx = fy   # ... and this is its cost
        elif self.iteration == self.max_iterations:
            return None
        elif fy <= self.fx:
            self.x, self.fx = self.y, fy
            self.d *= 0.95
        if self.y == self.left:
            self.fleft = fy
        elif self.y == self.right:
            self.fright = fy
        for _ in range(10_000):  # a boundary with a known cost is skipped; bounded so that a degenerate interval cannot spin
            y = self.clamp(self.x + self.uniform(-self.d, self.d))
            if (y == self.left and self.fleft is not None) or (y == self.right and self.fright is not None):
                continue
            break
        self.y = y
        return y

    def best(self) -> Tuple[float, float]:
        return self.x, self.fx
