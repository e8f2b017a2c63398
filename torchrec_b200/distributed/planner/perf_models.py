"""Plan-level perf models (cf. ``torchrec/distributed/planner/perf_models.py``)."""
from __future__ import annotations

from typing import List, cast

from torchrec_b200.distributed.planner.types import Perf, PerfModel, ShardingOption, Storage, Topology


class NoopPerfModel(PerfModel):
    """A plan is as slow as its most loaded rank."""

    def __init__(self, topology: Topology) -> None:
        self._topology = topology

    def rate(self, plan: List[ShardingOption]) -> float:
        perfs = [0.0] * self._topology.world_size
        for so in plan:
            for shard in so.shards:
                assert shard.rank is not None
                perfs[shard.rank] += cast(Perf, shard.perf).total
        return max(perfs)


class NoopStorageModel(PerfModel):
    """Rates a plan by the peak HBM of its fullest rank."""

    def __init__(self, topology: Topology) -> None:
        self._topology = topology

    def rate(self, plan: List[ShardingOption]) -> float:
        hbms = [0] * self._topology.world_size
        for so in plan:
            for shard in so.shards:
                assert shard.rank is not None
                hbms[shard.rank] += cast(Storage, shard.storage).hbm
        return max(hbms)
