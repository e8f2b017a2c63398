"""Planner data model: ``Perf``/``Storage``, ``Topology``, ``ShardingOption``/``Shard``,
``ParameterConstraints``, the plug-in ABCs and ``PlannerError``.

Counterpart of ``torchrec/distributed/planner/types.py:47-1147``.  The perf total differs on purpose:
for fused lookup+collective kernels compute and communication overlap, so a shard costs
``max(compute, comms)`` per direction instead of their sum.
"""
from __future__ import annotations

import abc
import hashlib
from copy import deepcopy
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Dict, List, Optional, Tuple, Union, cast

import torch
from torch import nn

from torchrec_b200.distributed.planner.constants import (
    BATCH_SIZE,
    BWD_COMPUTE_MULTIPLIER,
    CROSS_NODE_BANDWIDTH,
    DDR_CAP,
    DDR_MEM_BW,
    FUSED_DIST_OVERLAP,
    HBM_CAP,
    HBM_MEM_BW,
    HBM_TO_DDR_MEM_BW,
    INTRA_NODE_BANDWIDTH,
    POOLING_FACTOR,
    WEIGHTED_FEATURE_BWD_COMPUTE_MULTIPLIER,
)
from torchrec_b200.distributed.types import (
    BoundsCheckMode,
    CacheParams,
    KeyValueParams,
    ModuleSharder,
    ShardingPlan,
)
from torchrec_b200.modules.embedding_configs import DataType
from torchrec_b200.modules.embedding_modules import EmbeddingCollectionInterface


@dataclass(repr=True, eq=True)
class Perf:
    """Cost estimate (ms) of one shard per step."""

    fwd_compute: float
    fwd_comms: float
    bwd_compute: float
    bwd_comms: float
    prefetch_compute: float = 0.0

    @property
    def total(self) -> float:
        if FUSED_DIST_OVERLAP:
            return max(self.fwd_compute, self.fwd_comms) + max(self.bwd_compute, self.bwd_comms) + self.prefetch_compute
        return self.fwd_compute + self.bwd_compute + self.fwd_comms + self.bwd_comms + self.prefetch_compute

    def __add__(self, other: "Perf") -> "Perf":
        return Perf(self.fwd_compute + other.fwd_compute, self.fwd_comms + other.fwd_comms, self.bwd_compute + other.bwd_compute,
                    self.bwd_comms + other.bwd_comms, self.prefetch_compute + other.prefetch_compute)

    def __hash__(self) -> int:
        return hash((self.fwd_compute, self.fwd_comms, self.bwd_compute, self.bwd_comms, self.prefetch_compute))


@dataclass(repr=True, order=True, eq=True)
class Storage:
    hbm: int
    ddr: int

    def __add__(self, other: "Storage") -> "Storage":
        return Storage(hbm=self.hbm + other.hbm, ddr=self.ddr + other.ddr)

    def __sub__(self, other: "Storage") -> "Storage":
        return Storage(hbm=self.hbm - other.hbm, ddr=self.ddr - other.ddr)

    def __hash__(self) -> int:
        return hash((self.hbm, self.ddr))

    def fits_in(self, other: "Storage") -> bool:
        return self.hbm <= other.hbm and self.ddr <= other.ddr


@dataclass
class DeviceHardware:
    rank: int
    storage: Storage
    perf: Perf


class CustomTopologyData:
    """Per-rank overrides (``ddr_cap`` / ``hbm_cap``) for heterogeneous machines."""

    supported_fields = ["ddr_cap", "hbm_cap"]

    def __init__(self, data: Dict[str, List[int]], world_size: int) -> None:
        assert all(key in self.supported_fields for key in data.keys()), f"{data.keys()} not supported in CustomTopologyData"
        assert all(len(v) == world_size for v in data.values()), f"{data.values()} must be positive"
        self._data = data
        self._world_size = world_size

    def get_data(self, key: str) -> List[int]:
        assert key in self.supported_fields
        return self._data[key]

    def has_data(self, key: str) -> bool:
        return key in self._data


class CollectiveType(Enum):
    ALL_TO_ALL = "all_to_all"
    REDUCE_SCATTER = "reduce_scatter"
    ALL_GATHER = "all_gather"
    ALL_REDUCE = "all_reduce"


class GeneralizedCommsBandwidth(abc.ABC):
    @abc.abstractmethod
    def get_bw(self, local_world_size: int, world_size: int, collective_type: CollectiveType) -> float:
        ...

    @property
    @abc.abstractmethod
    def intra_host_bw(self) -> float:
        ...

    @property
    @abc.abstractmethod
    def inter_host_bw(self) -> float:
        ...


class BasicCommsBandwidths(GeneralizedCommsBandwidth):
    def __init__(self, inter_host_bw: float = CROSS_NODE_BANDWIDTH, intra_host_bw: float = INTRA_NODE_BANDWIDTH) -> None:
        self.name = "BasicCommsBandwidths"
        self._inter_host_bw = inter_host_bw
        self._intra_host_bw = intra_host_bw

    def __str__(self) -> str:
        return self.name + f": inter_host_bw={self.inter_host_bw}, intra_host_bw={self.intra_host_bw}"

    @property
    def inter_host_bw(self) -> float:
        return self._inter_host_bw

    @property
    def intra_host_bw(self) -> float:
        return self._intra_host_bw

    def get_bw(self, local_world_size: int, world_size: int, collective_type: CollectiveType) -> float:
        return self.intra_host_bw if world_size <= local_world_size else self.inter_host_bw


class Topology:
    """The machines a plan is made for: per-device storage and bandwidths."""

    def __init__(
        self,
        world_size: int,
        compute_device: str,
        hbm_cap: Optional[int] = None,
        ddr_cap: Optional[int] = None,
        local_world_size: Optional[int] = None,
        hbm_mem_bw: float = HBM_MEM_BW,
        ddr_mem_bw: float = DDR_MEM_BW,
        hbm_to_ddr_mem_bw: float = HBM_TO_DDR_MEM_BW,
        intra_host_bw: float = INTRA_NODE_BANDWIDTH,
        inter_host_bw: float = CROSS_NODE_BANDWIDTH,
        bwd_compute_multiplier: float = BWD_COMPUTE_MULTIPLIER,
        custom_topology_data: Optional[CustomTopologyData] = None,
        weighted_feature_bwd_compute_multiplier: float = WEIGHTED_FEATURE_BWD_COMPUTE_MULTIPLIER,
        uneven_sharding_perf_multiplier: float = 1.0,
        pod_size: Optional[int] = None,
        generalized_comms_bandwidths: Optional[GeneralizedCommsBandwidth] = None,
    ) -> None:
        assert compute_device in ["cpu", "cuda", "mtia"], f"unsupported compute device {compute_device}"
        self._compute_device = compute_device
        self._world_size = world_size
        hbm_per_device = [0] * world_size
        if self._compute_device == "cuda":
            hbm_per_device = [hbm_cap if hbm_cap else HBM_CAP] * world_size
        ddr_cap_per_rank = [ddr_cap if ddr_cap else DDR_CAP] * world_size
        if custom_topology_data:
            if custom_topology_data.has_data("hbm_cap"):
                hbm_per_device = custom_topology_data.get_data("hbm_cap")
            if custom_topology_data.has_data("ddr_cap"):
                ddr_cap_per_rank = custom_topology_data.get_data("ddr_cap")
        self._devices: List[DeviceHardware] = [
            DeviceHardware(rank=rank, storage=Storage(hbm=hbm_per_device[rank], ddr=ddr_cap_per_rank[rank]), perf=Perf(0, 0, 0, 0))
            for rank in range(world_size)
        ]
        self._local_world_size: int = local_world_size if local_world_size else world_size
        self._hbm_mem_bw = hbm_mem_bw
        self._ddr_mem_bw = ddr_mem_bw
        self._hbm_to_ddr_mem_bw = hbm_to_ddr_mem_bw
        self._comms_bandwidths: GeneralizedCommsBandwidth = generalized_comms_bandwidths or BasicCommsBandwidths(inter_host_bw, intra_host_bw)
        self._bwd_compute_multiplier = bwd_compute_multiplier
        self._custom_topology_data = custom_topology_data
        self._weighted_feature_bwd_compute_multiplier = weighted_feature_bwd_compute_multiplier
        self._uneven_sharding_perf_multiplier = uneven_sharding_perf_multiplier
        self._pod_size = pod_size if pod_size else self._local_world_size

    @property
    def compute_device(self) -> str:
        return self._compute_device

    @property
    def devices(self) -> List[DeviceHardware]:
        return self._devices

    @property
    def world_size(self) -> int:
        return self._world_size

    @property
    def local_world_size(self) -> int:
        return self._local_world_size

    @property
    def pod_size(self) -> int:
        return self._pod_size

    @property
    def hbm_mem_bw(self) -> float:
        return self._hbm_mem_bw

    @property
    def ddr_mem_bw(self) -> float:
        return self._ddr_mem_bw

    @property
    def hbm_to_ddr_mem_bw(self) -> float:
        return self._hbm_to_ddr_mem_bw

    @property
    def intra_host_bw(self) -> float:
        return self._comms_bandwidths.intra_host_bw

    @property
    def inter_host_bw(self) -> float:
        return self._comms_bandwidths.inter_host_bw

    @property
    def comms_bandwidths(self) -> GeneralizedCommsBandwidth:
        return self._comms_bandwidths

    @property
    def bwd_compute_multiplier(self) -> float:
        return self._bwd_compute_multiplier

    @property
    def weighted_feature_bwd_compute_multiplier(self) -> float:
        return self._weighted_feature_bwd_compute_multiplier

    @property
    def uneven_sharding_perf_multiplier(self) -> float:
        return self._uneven_sharding_perf_multiplier

    def __repr__(self) -> str:
        lines = [f"world_size={self._world_size}", f"compute_device={self._compute_device}", "devices="]
        lines += [f"\tdevice {i} {d}" for i, d in enumerate(self._devices)]
        lines += [f"local_world_size={self._local_world_size}", str(self._comms_bandwidths)]
        return "\n".join(lines) + "\n"

    def _hash(self) -> int:
        return hash_sha256_to_int(repr(self))


@dataclass
class Shard:
    size: List[int]
    offset: List[int]
    storage: Optional[Storage] = None
    perf: Optional[Perf] = None
    rank: Optional[int] = None

    def __hash__(self) -> int:
        return hash((tuple(self.size), tuple(self.offset), self.storage, self.perf, self.rank))

    def __str__(self) -> str:
        return f"Shard size: {tuple(self.size)}, offset: {tuple(self.offset)}, storage: {self.storage}, perf: {self.perf}, rank: {self.rank}"


class ShardingOption:
    """One way to shard one table: (sharding type, compute kernel) with its shards and estimates."""

    def __init__(
        self,
        name: str,
        tensor: torch.Tensor,
        module: Tuple[str, nn.Module],
        input_lengths: List[float],
        batch_size: int,
        sharding_type: str,
        partition_by: str,
        compute_kernel: str,
        shards: List[Shard],
        cache_params: Optional[CacheParams] = None,
        enforce_hbm: Optional[bool] = None,
        stochastic_rounding: Optional[bool] = None,
        bounds_check_mode: Optional[BoundsCheckMode] = None,
        dependency: Optional[str] = None,
        is_pooled: Optional[bool] = None,
        feature_names: Optional[List[str]] = None,
        output_dtype: Optional[DataType] = None,
        key_value_params: Optional[KeyValueParams] = None,
    ) -> None:
        self.name = name
        self._tensor = tensor
        self._module = module
        self.input_lengths = input_lengths
        self.batch_size = batch_size
        self.sharding_type = sharding_type
        self.partition_by = partition_by
        self.compute_kernel = compute_kernel
        self.shards = shards
        self.cache_params = cache_params
        self.enforce_hbm = enforce_hbm
        self.stochastic_rounding = stochastic_rounding
        self.bounds_check_mode = bounds_check_mode
        self.dependency = dependency
        self._is_pooled = is_pooled
        self.is_weighted: Optional[bool] = None
        self.feature_names: Optional[List[str]] = feature_names
        self.output_dtype: Optional[DataType] = output_dtype
        self.key_value_params: Optional[KeyValueParams] = key_value_params

    @property
    def tensor(self) -> torch.Tensor:
        return self._tensor

    @property
    def module(self) -> Tuple[str, nn.Module]:
        return self._module

    @property
    def fqn(self) -> str:
        return self.module[0] + "." + self.name

    @property
    def cache_load_factor(self) -> Optional[float]:
        return self.cache_params.load_factor if self.cache_params is not None else None

    @property
    def path(self) -> str:
        return self.module[0]

    @property
    def num_shards(self) -> int:
        return len(self.shards)

    @property
    def num_inputs(self) -> int:
        return len(self.input_lengths)

    @property
    def total_storage(self) -> Storage:
        storage = Storage(hbm=0, ddr=0)
        for shard in self.shards:
            storage += cast(Storage, shard.storage)
        return storage

    @property
    def total_perf(self) -> float:
        return sum(cast(Perf, shard.perf).total for shard in self.shards)

    @property
    def is_pooled(self) -> bool:
        if self._is_pooled is None:
            self._is_pooled = ShardingOption.module_pooled(self.module[1], self.name)
        return self._is_pooled

    @staticmethod
    def module_pooled(module: nn.Module, sharding_option_name: str) -> bool:
        if isinstance(module, EmbeddingCollectionInterface) or type(module).__name__.endswith("EmbeddingCollection") and "Bag" not in type(module).__name__:
            return False
        for submodule in module.modules():
            if isinstance(submodule, EmbeddingCollectionInterface):
                for name, _ in submodule.named_parameters():
                    if sharding_option_name in name:
                        return False
        return True

    def __hash__(self) -> int:
        return hash((self.fqn, self.sharding_type, self.compute_kernel, tuple(self.shards), self.cache_params))

    def __deepcopy__(self, memo: Optional[Dict[int, "ShardingOption"]]) -> "ShardingOption":
        cls = self.__class__
        result = cls.__new__(cls)
        for k, v in self.__dict__.items():
            if k in ("_tensor", "_module"):
                setattr(result, k, v)
            else:
                setattr(result, k, deepcopy(v, memo))
        return result

    def __str__(self) -> str:
        return "\n".join(f"{k}: {v}" for k, v in self.__dict__.items() if k not in ("_tensor", "_module"))


class PartitionByType(Enum):
    DEVICE = "device"
    HOST = "host"
    UNIFORM = "uniform"
    MULTI_HOST = "multi_host"


@dataclass
class ParameterConstraints:
    """User restrictions on how a table may be sharded, plus the statistics the estimators use
    (``pooling_factors``: mean ids per sample per feature; ``num_poolings``; ``batch_sizes``)."""

    sharding_types: Optional[List[str]] = None
    compute_kernels: Optional[List[str]] = None
    min_partition: Optional[int] = None
    pooling_factors: List[float] = field(default_factory=lambda: [POOLING_FACTOR])
    num_poolings: Optional[List[float]] = None
    batch_sizes: Optional[List[int]] = None
    is_weighted: bool = False
    cache_params: Optional[CacheParams] = None
    enforce_hbm: Optional[bool] = None
    stochastic_rounding: Optional[bool] = None
    bounds_check_mode: Optional[BoundsCheckMode] = None
    feature_names: Optional[List[str]] = None
    output_dtype: Optional[DataType] = None
    device_group: Optional[str] = None
    key_value_params: Optional[KeyValueParams] = None

    def __hash__(self) -> int:
        return hash_sha256_to_int(repr(self))


class PlannerErrorType(Enum):
    INSUFFICIENT_STORAGE = "insufficient_storage"
    STRICT_CONSTRAINTS = "strict_constraints"
    PARTITION = "partition"
    OTHER = "other"
    PLANNER_INPUT_CONTEXT_MISMATCH = "planner_input_context_mismatch"
    PLAN_LOADING_FAILED = "plan_loading_failed"


class PlannerError(Exception):
    def __init__(self, message: str, error_type: PlannerErrorType = PlannerErrorType.OTHER) -> None:
        self.error_type = error_type
        super().__init__(message)


# ---- plug-in interfaces ------------------------------------------------------------------------------
class StorageReservation(abc.ABC):
    """Sets aside memory for dense parameters, inputs and a safety margin before tables are placed."""

    @abc.abstractmethod
    def reserve(self, topology: Topology, batch_size: int, module: nn.Module, sharders: List[ModuleSharder[nn.Module]],
                constraints: Optional[Dict[str, ParameterConstraints]] = None) -> Topology:
        ...

    @property
    @abc.abstractmethod
    def last_reserved_topology(self) -> Optional[Topology]:
        ...


class PerfModel(abc.ABC):
    @abc.abstractmethod
    def rate(self, plan: List[ShardingOption]) -> float:
        ...


class ShardEstimator(abc.ABC):
    @abc.abstractmethod
    def __init__(self, topology: Topology, constraints: Optional[Dict[str, ParameterConstraints]] = None) -> None:
        ...

    @abc.abstractmethod
    def estimate(self, sharding_options: List[ShardingOption], sharder_map: Optional[Dict[str, ModuleSharder[nn.Module]]] = None) -> None:
        ...


class Enumerator(abc.ABC):
    @abc.abstractmethod
    def __init__(self, topology: Topology, batch_size: int = BATCH_SIZE, constraints: Optional[Dict[str, ParameterConstraints]] = None,
                 estimator: Optional[Union[ShardEstimator, List[ShardEstimator]]] = None) -> None:
        ...

    @abc.abstractmethod
    def enumerate(self, module: nn.Module, sharders: List[ModuleSharder[nn.Module]]) -> List[ShardingOption]:
        ...

    @abc.abstractmethod
    def populate_estimates(self, sharding_options: List[ShardingOption]) -> None:
        ...


class Proposer(abc.ABC):
    """Proposes complete plans (one option per table); ``feedback`` tells it how the last one did."""

    @abc.abstractmethod
    def load(self, search_space: List[ShardingOption], enumerator: Optional[Enumerator] = None) -> None:
        ...

    @abc.abstractmethod
    def feedback(self, partitionable: bool, plan: Optional[List[ShardingOption]] = None, perf_rating: Optional[float] = None,
                 storage_constraint: Optional[Topology] = None) -> None:
        ...

    @abc.abstractmethod
    def propose(self) -> Optional[List[ShardingOption]]:
        ...


class Partitioner(abc.ABC):
    """Places the shards of a proposal on devices within the storage constraint."""

    @abc.abstractmethod
    def partition(self, proposal: List[ShardingOption], storage_constraint: Topology) -> List[ShardingOption]:
        ...


class Stats(abc.ABC):
    @abc.abstractmethod
    def log(self, sharding_plan: ShardingPlan, topology: Topology, batch_size: int, storage_reservation: StorageReservation, num_proposals: int,
            num_plans: int, run_time: float, best_plan: List[ShardingOption], constraints: Optional[Dict[str, ParameterConstraints]] = None,
            sharders: Optional[List[ModuleSharder[nn.Module]]] = None, enumerator: Optional[Enumerator] = None, debug: bool = False) -> None:
        ...


def hash_sha256_to_int(hashable_list: Any) -> int:
    serialized = str(hashable_list).encode("utf-8")
    return int(hashlib.sha256(serialized).hexdigest(), 16)


def hash_sha256_str(hashable_list: Any) -> str:
    return hashlib.sha256(str(hashable_list).encode("utf-8")).hexdigest()


def hash_planner_context_inputs(topology: Topology, batch_size: int, enumerator: Enumerator, storage_reservation: StorageReservation,
                                constraints: Optional[Dict[str, ParameterConstraints]], hash_function=hash_sha256_to_int):
    """Fingerprint of everything that determines a plan; used to validate a loaded plan."""
    assert hasattr(enumerator, "last_stored_search_space"), "This enumerator is not compatible with hashing"
    search_space = enumerator.last_stored_search_space  # type: ignore[attr-defined]
    storage_constraint = storage_reservation.last_reserved_topology
    hashable = [
        topology, batch_size,
        [[so.fqn, so.sharding_type, so.compute_kernel, tuple(so.shards), so.cache_params] for so in search_space],
        storage_constraint, storage_reservation._last_reserved_topology if hasattr(storage_reservation, "_last_reserved_topology") else None,
        sorted(constraints.items()) if constraints else None,
    ]
    return hash_function(hashable)
