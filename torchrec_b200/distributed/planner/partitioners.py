"""Partitioners: assign the shards of a proposal to ranks.

``GreedyPerfPartitioner`` sorts options by cost and repeatedly gives the next one to the least
loaded device (or node / all devices, depending on the sharding type) that still has room;
``MemoryBalancedPartitioner`` then re-partitions under progressively tighter memory caps to find a
plan with lower peak memory at (almost) the same perf.
Counterpart of ``torchrec/distributed/planner/partitioners.py``.
"""
from __future__ import annotations

import copy
import heapq
import logging
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple, cast

from torchrec_b200.distributed.planner.perf_models import NoopPerfModel
from torchrec_b200.distributed.planner.types import (
    DeviceHardware,
    PartitionByType,
    Partitioner,
    Perf,
    PerfModel,
    PlannerError,
    PlannerErrorType,
    ShardingOption,
    Storage,
    Topology,
)
from torchrec_b200.distributed.planner.utils import bytes_to_gb, reset_shard_rank
from torchrec_b200.distributed.types import ShardingType

logger: logging.Logger = logging.getLogger(__name__)


def _sort_devices_by_perf(devices: List[List[DeviceHardware]]) -> List[List[DeviceHardware]]:
    def _get_perf_sum(device_list: List[DeviceHardware]) -> float:
        return sum(d.perf.total for d in device_list)

    return sorted(devices, key=_get_perf_sum)


def _get_uniform_sharding_options(sharding_options: List[ShardingOption]) -> List[ShardingOption]:
    return [so for so in sharding_options if so.partition_by == PartitionByType.UNIFORM.value]


@dataclass
class ShardingOptionGroup:
    sharding_options: List[ShardingOption]
    storage_sum: Storage
    perf_sum: float
    param_count: int


class SortBy:
    STORAGE = "storage"
    PERF = "perf"


def _group_and_sort_non_uniform_sharding_options(sharding_options: List[ShardingOption], sort_by: str = SortBy.STORAGE,
                                                 balance_modules: bool = False) -> List[ShardingOptionGroup]:
    groups_by_dep: Dict[str, ShardingOptionGroup] = {}
    for so in sharding_options:
        if so.partition_by == PartitionByType.UNIFORM.value:
            continue
        key = so.dependency or so.fqn
        if key not in groups_by_dep:
            groups_by_dep[key] = ShardingOptionGroup([so], so.total_storage, so.total_perf, 1)
        else:
            g = groups_by_dep[key]
            g.sharding_options.append(so)
            g.storage_sum += so.total_storage
            g.perf_sum += so.total_perf
    groups = list(groups_by_dep.values())
    if sort_by == SortBy.STORAGE:
        groups.sort(key=lambda g: (g.storage_sum.hbm, g.perf_sum), reverse=True)
    else:
        groups.sort(key=lambda g: (g.perf_sum, g.storage_sum.hbm), reverse=True)
    return groups


@dataclass
class OrderedDeviceHardware:
    """A device as the greedy partitioner's heap orders it: least loaded first; among equally loaded devices the lower local rank
    first, so that consecutive shards spread over the hosts (and their DDR) instead of filling one host
    (``torchrec/distributed/planner/partitioners.py:158-173``)."""

    device: DeviceHardware
    local_world_size: int

    def _key(self) -> Tuple[float, int, int]:
        return (self.device.perf.total, self.device.rank % self.local_world_size, self.device.rank)

    def __lt__(self, other: "OrderedDeviceHardware") -> bool:
        return self._key() < other._key()


class GreedyPerfPartitioner(Partitioner):
    def __init__(self, sort_by: str = SortBy.STORAGE, balance_modules: bool = False) -> None:
        self._sort_by = sort_by
        self._balance_modules = balance_modules

    def partition(self, proposal: List[ShardingOption], storage_constraint: Topology) -> List[ShardingOption]:
        _topology = copy.deepcopy(storage_constraint)
        minheap_devices: Optional[List] = None
        _host_level_devices = self._get_host_level_devices(_topology)
        # uniform options first: they take the same amount from every device
        for so in _get_uniform_sharding_options(proposal):
            self._uniform_partition([so], _topology.devices)
        for group in _group_and_sort_non_uniform_sharding_options(proposal, sort_by=self._sort_by, balance_modules=self._balance_modules):
            pb = group.sharding_options[0].partition_by
            if pb == PartitionByType.MULTI_HOST.value:
                self._multi_hosts_partition(group, _host_level_devices)
                minheap_devices = None
            elif pb == PartitionByType.HOST.value:
                self._cohost_partition(group, _host_level_devices)
                minheap_devices = None
            elif pb == PartitionByType.DEVICE.value:
                if minheap_devices is None:
                    minheap_devices = self._establish_minheap(_topology.devices, _topology.local_world_size)
                assert len(group.sharding_options) == 1 or all(so.dependency for so in group.sharding_options), "Unexpected length for sharding options"
                self._device_partition(group, minheap_devices)
            else:
                raise RuntimeError(f"Unexpected sharding option group {group}")
        self._topology = _topology
        return proposal

    @staticmethod
    def _establish_minheap(devices: List[DeviceHardware], local_world_size: int) -> List:
        heap = [OrderedDeviceHardware(d, max(local_world_size, 1)) for d in devices]
        heapq.heapify(heap)
        return heap

    @classmethod
    def _device_partition(cls, group: ShardingOptionGroup, minheap_devices: List, bulk_heapify_threshold: float = 0.25) -> None:
        for so in group.sharding_options:
            for shard in so.shards:
                tmp = []
                placed = False
                while minheap_devices:
                    entry = heapq.heappop(minheap_devices)
                    device = entry.device
                    storage = cast(Storage, shard.storage)
                    if storage.fits_in(device.storage):
                        shard.rank = device.rank
                        device.storage -= storage
                        device.perf += cast(Perf, shard.perf)
                        heapq.heappush(minheap_devices, entry)
                        placed = True
                        break
                    tmp.append(entry)
                for t in tmp:
                    heapq.heappush(minheap_devices, t)
                if not placed:
                    raise PlannerError(
                        error_type=PlannerErrorType.PARTITION,
                        message=f"Device partition failed. Couldn't find a rank for shard {shard} of table {so.name}, largest device storage: "
                                f"{max((e.device.storage for e in minheap_devices), key=lambda s: s.hbm) if minheap_devices else None}",
                    )

    @classmethod
    def _cohost_partition(cls, group: ShardingOptionGroup, _host_level_devices: List[List[DeviceHardware]]) -> None:
        sorted_hosts = _sort_devices_by_perf(_host_level_devices)
        for devices in sorted_hosts:
            host_devices = copy.deepcopy(devices)
            host_storage = Storage(hbm=0, ddr=0)
            for d in host_devices:
                host_storage += d.storage
            if not group.storage_sum.fits_in(host_storage):
                continue
            success = True
            minheap = cls._establish_minheap(host_devices, len(host_devices))
            for so in group.sharding_options:
                try:
                    if so.sharding_type == ShardingType.TABLE_ROW_WISE.value:
                        cls._uniform_partition([so], host_devices)
                        minheap = cls._establish_minheap(host_devices, len(host_devices))
                    elif so.sharding_type == ShardingType.TABLE_COLUMN_WISE.value:
                        cls._device_partition(ShardingOptionGroup([so], so.total_storage, so.total_perf, 1), minheap)
                    else:
                        raise RuntimeError(f"unexpected cohost sharding type: {so.sharding_type}")
                except PlannerError:
                    success = False
                    break
            if success:
                for d, nd in zip(devices, host_devices):
                    d.storage, d.perf = nd.storage, nd.perf
                return
        raise PlannerError(error_type=PlannerErrorType.PARTITION, message=f"can't find a host for sharding option group {[so.name for so in group.sharding_options]}")

    @classmethod
    def _multi_hosts_partition(cls, group: ShardingOptionGroup, _host_level_devices: List[List[DeviceHardware]]) -> None:
        so = group.sharding_options[0]
        local = len(_host_level_devices[0])
        host_index, host_devices = 0, None
        sorted_hosts = _sort_devices_by_perf(_host_level_devices)
        for s in range(0, len(so.shards), local):
            shards = so.shards[s: s + local]
            if host_index >= len(sorted_hosts):
                raise PlannerError(error_type=PlannerErrorType.PARTITION, message=f"not enough hosts for grid sharding of {so.name}")
            host_devices = sorted_hosts[host_index]
            host_index += 1
            for shard, device in zip(shards, host_devices):
                storage = cast(Storage, shard.storage)
                if not storage.fits_in(device.storage):
                    raise PlannerError(error_type=PlannerErrorType.PARTITION, message=f"grid shard {shard} of {so.name} does not fit on rank {device.rank}")
                shard.rank = device.rank
                device.storage -= storage
                device.perf += cast(Perf, shard.perf)

    @staticmethod
    def _get_host_level_devices(_topology: Topology) -> List[List[DeviceHardware]]:
        n_hosts = _topology.world_size // _topology.local_world_size
        return [_topology.devices[i * _topology.local_world_size: (i + 1) * _topology.local_world_size] for i in range(n_hosts)]

    @staticmethod
    def _uniform_partition(sharding_options: List[ShardingOption], devices: List[DeviceHardware]) -> None:
        for so in sharding_options:
            if so.num_shards != len(devices):
                raise PlannerError(error_type=PlannerErrorType.PARTITION, message=f"For a uniform partition, the number of shards ({so.num_shards}) must equal the number of devices ({len(devices)})")
            for i in range(len(devices)):
                storage_needed = cast(Storage, so.shards[i].storage)
                if not storage_needed.fits_in(devices[i].storage):
                    raise PlannerError(error_type=PlannerErrorType.PARTITION, message=f"Shard of size {storage_needed} bytes does not fit on any rank. Device memory cap: {devices[i].storage}.")
                so.shards[i].rank = devices[i].rank
                devices[i].storage -= storage_needed
                devices[i].perf += cast(Perf, so.shards[i].perf)


class MemoryBalancedPartitioner(Partitioner):
    """Wraps the greedy partitioner: search for the smallest HBM cap that keeps perf within ``tolerance``."""

    def __init__(self, max_search_count: int = 10, tolerance: float = 0.02, balance_modules: bool = False) -> None:
        self._max_search_count = max_search_count
        self._tolerance = tolerance
        self._balance_modules = balance_modules

    def partition(self, proposal: List[ShardingOption], storage_constraint: Topology) -> List[ShardingOption]:
        greedy = GreedyPerfPartitioner(sort_by=SortBy.PERF, balance_modules=self._balance_modules)
        default_plan = copy.deepcopy(greedy.partition(proposal, storage_constraint))
        original_total_hbm = sum(d.storage.hbm for d in storage_constraint.devices)
        if original_total_hbm == 0:
            return default_plan
        perf_model: PerfModel = NoopPerfModel(storage_constraint)
        default_perf = perf_model.rate(default_plan)
        max_hbm_per_device = max(d.storage.hbm for d in storage_constraint.devices)
        hbm_requirement = sum(so.total_storage.hbm for so in proposal)
        min_hbm_per_device = int(hbm_requirement / len(storage_constraint.devices))
        best_plan = default_plan
        lo, hi = min_hbm_per_device, max_hbm_per_device
        for _ in range(self._max_search_count):
            mid = (lo + hi) // 2
            constraint = copy.deepcopy(storage_constraint)
            for d in constraint.devices:
                d.storage.hbm = min(d.storage.hbm, mid)
            try:
                reset_shard_rank(proposal)
                plan = copy.deepcopy(greedy.partition(proposal, constraint))
                perf = perf_model.rate(plan)
                if perf <= default_perf * (1 + self._tolerance):
                    best_plan = plan
                    hi = mid
                else:
                    lo = mid
            except PlannerError:
                lo = mid
        # copy the chosen ranks back into the caller's options
        for so, best in zip(proposal, best_plan):
            for shard, bshard in zip(so.shards, best.shards):
                shard.rank = bshard.rank
        return best_plan
