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


_PERF_FIELDS = ("fwd_compute", "fwd_comms", "bwd_compute", "bwd_comms", "prefetch_compute")


@dataclass(repr=True, eq=True)
class Perf:
    """Cost estimate (ms) of one shard per step."""

    fwd_compute: float
    fwd_comms: float
    bwd_compute: float
    bwd_comms: float
    prefetch_compute: float = 0.0

    def _tuple(self) -> Tuple[float, ...]:
        return tuple(getattr(self, f) for f in _PERF_FIELDS)

    @property
    def total(self) -> float:
        fc, fx, bc, bx, pre = self._tuple()
        if FUSED_DIST_OVERLAP:
            # the exchange runs inside the lookup kernels: per direction the slower of the two sets the time
            return max(fc, fx) + max(bc, bx) + pre
        return fc + fx + bc + bx + pre

    def __add__(self, other: "Perf") -> "Perf":
        return Perf(*(a + b for a, b in zip(self._tuple(), other._tuple())))

    def __hash__(self) -> int:
        return hash(self._tuple())


@dataclass(repr=True, order=True, eq=True)
class Storage:
    hbm: int
    ddr: int

    def __add__(self, other: "Storage") -> "Storage":
        return Storage(self.hbm + other.hbm, self.ddr + other.ddr)

    def __sub__(self, other: "Storage") -> "Storage":
        return Storage(self.hbm - other.hbm, self.ddr - other.ddr)

    def __hash__(self) -> int:
        return hash((self.hbm, self.ddr))

    def fits_in(self, other: "Storage") -> bool:
        return other.hbm >= self.hbm and other.ddr >= self.ddr


@dataclass
class DeviceHardware:
    rank: int
    storage: Storage
    perf: Perf


class CustomTopologyData:
    """Per-rank overrides (``ddr_cap`` / ``hbm_cap``) for heterogeneous machines."""

    supported_fields = ["ddr_cap", "hbm_cap"]

    def __init__(self, data: Dict[str, List[int]], world_size: int) -> None:
        unknown = [k for k in data if k not in self.supported_fields]
        assert not unknown, f"{data.keys()} not supported in CustomTopologyData"
        short = [k for k, v in data.items() if len(v) != world_size]
        assert not short, f"{data.values()} must be positive"
        self._data, self._world_size = data, world_size

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
    """Two numbers: what a collective gets inside a node and what it gets across nodes."""

    def __init__(self, inter_host_bw: float = CROSS_NODE_BANDWIDTH, intra_host_bw: float = INTRA_NODE_BANDWIDTH) -> None:
        self.name = type(self).__name__
        self._bw = {"inter": inter_host_bw, "intra": intra_host_bw}

    def __str__(self) -> str:
        return f"{self.name}: inter_host_bw={self.inter_host_bw}, intra_host_bw={self.intra_host_bw}"

    @property
    def inter_host_bw(self) -> float:
        return self._bw["inter"]

    @property
    def intra_host_bw(self) -> float:
        return self._bw["intra"]

    def get_bw(self, local_world_size: int, world_size: int, collective_type: CollectiveType) -> float:
        spans_nodes = world_size > local_world_size
        return self._bw["inter" if spans_nodes else "intra"]


def _read_only(attr: str):
    return property(lambda self: getattr(self, attr))


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
        self._compute_device, self._world_size = compute_device, world_size
        self._custom_topology_data = custom_topology_data

        def per_rank(key: str, uniform: int) -> List[int]:
            if custom_topology_data is not None and custom_topology_data.has_data(key):
                return custom_topology_data.get_data(key)
            return [uniform] * world_size

        hbm = per_rank("hbm_cap", (hbm_cap or HBM_CAP) if compute_device == "cuda" else 0)
        ddr = per_rank("ddr_cap", ddr_cap or DDR_CAP)
        self._devices: List[DeviceHardware] = [DeviceHardware(r, Storage(hbm=hbm[r], ddr=ddr[r]), Perf(0, 0, 0, 0)) for r in range(world_size)]
        self._local_world_size: int = local_world_size or world_size
        self._pod_size = pod_size or self._local_world_size
        self._hbm_mem_bw, self._ddr_mem_bw, self._hbm_to_ddr_mem_bw = hbm_mem_bw, ddr_mem_bw, hbm_to_ddr_mem_bw
        self._comms_bandwidths: GeneralizedCommsBandwidth = generalized_comms_bandwidths or BasicCommsBandwidths(inter_host_bw, intra_host_bw)
        self._bwd_compute_multiplier = bwd_compute_multiplier
        self._weighted_feature_bwd_compute_multiplier = weighted_feature_bwd_compute_multiplier
        self._uneven_sharding_perf_multiplier = uneven_sharding_perf_multiplier

    compute_device = _read_only("_compute_device")
    devices = _read_only("_devices")
    world_size = _read_only("_world_size")
    local_world_size = _read_only("_local_world_size")
    pod_size = _read_only("_pod_size")
    hbm_mem_bw = _read_only("_hbm_mem_bw")
    ddr_mem_bw = _read_only("_ddr_mem_bw")
    hbm_to_ddr_mem_bw = _read_only("_hbm_to_ddr_mem_bw")
    comms_bandwidths = _read_only("_comms_bandwidths")
    bwd_compute_multiplier = _read_only("_bwd_compute_multiplier")
    weighted_feature_bwd_compute_multiplier = _read_only("_weighted_feature_bwd_compute_multiplier")
    uneven_sharding_perf_multiplier = _read_only("_uneven_sharding_perf_multiplier")

    @property
    def intra_host_bw(self) -> float:
        return self._comms_bandwidths.intra_host_bw

    @property
    def inter_host_bw(self) -> float:
        return self._comms_bandwidths.inter_host_bw

    def __repr__(self) -> str:
        device_lines = [f"\tdevice {i} {d}" for i, d in enumerate(self._devices)]
        head = [f"world_size={self._world_size}", f"compute_device={self._compute_device}", "devices="]
        tail = [f"local_world_size={self._local_world_size}", str(self._comms_bandwidths)]
        return "\n".join(head + device_lines + tail) + "\n"

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
        return hash((*self.size, -1, *self.offset, self.storage, self.perf, self.rank))

    def __str__(self) -> str:
        return f"Shard size: {tuple(self.size)}, offset: {tuple(self.offset)}, storage: {self.storage}, perf: {self.perf}, rank: {self.rank}"


_NOT_COPIED = ("_tensor", "_module")  # shared with the model: a deep copy of an option must not clone them


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
        given = dict(locals())
        for private in ("tensor", "module", "is_pooled"):
            setattr(self, "_" + private, given.pop(private))
        given.pop("self")
        self.__dict__.update(given)
        self.is_weighted: Optional[bool] = None

    @property
    def tensor(self) -> torch.Tensor:
        return self._tensor

    @property
    def module(self) -> Tuple[str, nn.Module]:
        return self._module

    @property
    def path(self) -> str:
        return self._module[0]

    @property
    def fqn(self) -> str:
        return f"{self.path}.{self.name}"

    @property
    def cache_load_factor(self) -> Optional[float]:
        cp = self.cache_params
        return None if cp is None else cp.load_factor

    @property
    def num_shards(self) -> int:
        return len(self.shards)

    @property
    def num_inputs(self) -> int:
        return len(self.input_lengths)

    @property
    def total_storage(self) -> Storage:
        return Storage(hbm=sum(cast(Storage, s.storage).hbm for s in self.shards), ddr=sum(cast(Storage, s.storage).ddr for s in self.shards))

    @property
    def total_perf(self) -> float:
        return sum(cast(Perf, s.perf).total for s in self.shards)

    @property
    def is_pooled(self) -> bool:
        if self._is_pooled is None:
            self._is_pooled = self.module_pooled(self._module[1], self.name)
        return self._is_pooled

    @staticmethod
    def module_pooled(module: nn.Module, sharding_option_name: str) -> bool:
        """False when the table belongs to an (unpooled) embedding collection, directly or through a wrapper module."""
        kind = type(module).__name__
        if isinstance(module, EmbeddingCollectionInterface) or (kind.endswith("EmbeddingCollection") and "Bag" not in kind):
            return False
        for sub in module.modules():
            if isinstance(sub, EmbeddingCollectionInterface) and any(sharding_option_name in n for n, _ in sub.named_parameters()):
                return False
        return True

    def __hash__(self) -> int:
        return hash((self.fqn, self.sharding_type, self.compute_kernel, tuple(self.shards), self.cache_params))

    def storage_hash(self) -> int:
        """Key of this option in a stored plan: stable across processes (no salted ``hash``), and a function only of what the
        enumerator decides before any placement - table, sharding type, kernel, cache load factor, number of shards
        (``torchrec/distributed/planner/types.py:641-655``)."""
        text = f"{self.fqn}|{self.sharding_type}|{self.compute_kernel}|{self.cache_load_factor}|{self.num_shards}"
        return int.from_bytes(hashlib.blake2b(text.encode("utf-8"), digest_size=7).digest(), "big")

    def __deepcopy__(self, memo: Optional[Dict[int, "ShardingOption"]]) -> "ShardingOption":
        clone = object.__new__(type(self))
        clone.__dict__.update({k: (v if k in _NOT_COPIED else deepcopy(v, memo)) for k, v in self.__dict__.items()})
        return clone

    def __str__(self) -> str:
        return "\n".join(f"{k}: {v}" for k, v in self.__dict__.items() if k not in _NOT_COPIED)


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


def hash_sha256_str(hashable_list: Any) -> str:
    return hashlib.sha256(str(hashable_list).encode("utf-8")).hexdigest()


def hash_sha256_to_int(hashable_list: Any) -> int:
    return int(hash_sha256_str(hashable_list), 16)


def hash_planner_context_inputs(topology: Topology, batch_size: int, enumerator: Enumerator, storage_reservation: StorageReservation,
                                constraints: Optional[Dict[str, ParameterConstraints]], hash_function=hash_sha256_to_int):
    """Fingerprint of everything that determines a plan; used to validate a loaded plan."""
    assert hasattr(enumerator, "last_stored_search_space"), "This enumerator is not compatible with hashing"
    options = [[o.fqn, o.sharding_type, o.compute_kernel, tuple(o.shards), o.cache_params] for o in enumerator.last_stored_search_space]  # type: ignore[attr-defined]
    reserved = storage_reservation.last_reserved_topology
    return hash_function([topology, batch_size, options, reserved, getattr(storage_reservation, "_last_reserved_topology", None),
                          sorted(constraints.items()) if constraints else None])


def hash_planner_context_inputs_str(topology: Topology, batch_size: int, enumerator: Enumerator, storage_reservation: StorageReservation,
                                    constraints: Optional[Dict[str, ParameterConstraints]], hash_function=hash_sha256_str) -> str:
    """The same fingerprint as ``hash_planner_context_inputs``, as a hex string (what a stored plan carries)."""
    return hash_planner_context_inputs(topology, batch_size, enumerator, storage_reservation, constraints, hash_function=hash_function)


class PlanLoader(abc.ABC):
    """Source of a plan computed earlier (to skip planning, or as the starting point of the next search).  ``load`` returns the stored
    sharding options keyed by the hash of the enumerated option they stand for; ``plan_context_hash`` the fingerprint of the inputs
    the stored plan was computed for, so that a loader can refuse a plan made for another model or topology."""

    @abc.abstractmethod
    def load(self) -> Optional[Dict[int, "ShardingOption"]]:
        ...

    @abc.abstractmethod
    def plan_context_hash(self) -> Optional[str]:
        ...

    def get_plan_id(self) -> Optional[str]:
        """Name of the stored plan for messages (optional)."""
        return None


@dataclass
class CriticalPathEstimate:
    """Time of the slowest rank, split into exchange and compute."""

    comms_estimate: float
    comp_estimate: float

    def total(self) -> float:
        return self.comms_estimate + self.comp_estimate


@dataclass
class PlanDebugStats:
    """What a planner reports about itself next to the plan (for logging)."""

    planner_type: str
    timeout_seconds: Optional[int]
