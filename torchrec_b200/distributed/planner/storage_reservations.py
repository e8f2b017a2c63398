"""Storage reservations: memory set aside before tables are placed
(cf. ``torchrec/distributed/planner/storage_reservations.py``)."""
from __future__ import annotations

import copy
import logging
import math
from typing import Dict, List, Optional, Set, Tuple

from torch import nn

from torchrec_b200.distributed.planner.constants import BIGINT_DTYPE, POOLING_FACTOR
from torchrec_b200.distributed.planner.types import ParameterConstraints, PlannerError, PlannerErrorType, Storage, StorageReservation, Topology
from torchrec_b200.distributed.planner.utils import sharder_name, storage_repr_in_gb
from torchrec_b200.distributed.types import ModuleSharder, get_tensor_size_bytes

logger: logging.Logger = logging.getLogger(__name__)


def _get_module_size(module: nn.Module, multiplier: float) -> int:
    parameters_size = sum(multiplier * p.element_size() * p.nelement() for p in module.parameters())
    buffers_size = sum(b.element_size() * b.nelement() for b in module.buffers())
    return round(parameters_size + buffers_size)


def _get_dense_tensor_size(module: nn.Module, shardable_modules: Set[nn.Module], multiplier: float = 6.0) -> int:
    """Bytes of the unsharded part: weights + gradients + optimizer state + DDP buckets ~= 6x weights."""
    dense_tensor_size = _get_module_size(module, multiplier) - sum(_get_module_size(m, multiplier) for m in shardable_modules)
    return max(dense_tensor_size, 0)


def _reserve_dense_storage(topology: Topology, module: nn.Module, shardable_modules: Set[nn.Module], multiplier: float, dense_tensor_estimate: Optional[int] = None) -> Storage:
    dense_tensor_size = _get_dense_tensor_size(module, shardable_modules, multiplier)
    if dense_tensor_estimate:
        dense_tensor_size = dense_tensor_estimate
    dense_tensor_storage = Storage(hbm=dense_tensor_size if topology.compute_device == "cuda" else 0, ddr=dense_tensor_size if topology.compute_device in {"cpu", "mtia"} else 0)
    for device in topology.devices:
        device.storage -= dense_tensor_storage
    return dense_tensor_storage


def _get_batch_inputs_and_shardable_parameters(module: nn.Module, sharders: List[ModuleSharder[nn.Module]], batch_size: int,
                                               constraints: Optional[Dict[str, ParameterConstraints]] = None) -> Tuple[List[float], Set[nn.Module]]:
    sharder_map = {sharder_name(s.module_type): s for s in sharders}
    input_lengths: List[float] = []
    batch_sizes: List[int] = []
    shardable_modules: Set[nn.Module] = set()

    def populate(m: nn.Module) -> None:
        sharder = sharder_map.get(sharder_name(type(m)), None)
        if sharder:
            names = sharder.shardable_parameters(m).keys()
            shardable_modules.add(m)
            for name in names:
                pooling = constraints[name].pooling_factors if constraints and constraints.get(name) else [POOLING_FACTOR]
                input_lengths.extend(pooling)
                bs = constraints[name].batch_sizes if constraints and constraints.get(name) and constraints[name].batch_sizes else [batch_size] * len(pooling)
                batch_sizes.extend(bs)
        else:
            for c in m.children():
                populate(c)

    populate(module)
    batch_inputs = [l * b for l, b in zip(input_lengths, batch_sizes)]
    return batch_inputs, shardable_modules


def _reserve_kjt_storage(topology: Topology, batch_size: int, batch_inputs: List[float], input_data_type_size: int, multiplier: int) -> Storage:
    kjt_size = math.ceil(sum(batch_inputs) * float(input_data_type_size)) * multiplier
    kjt_storage = Storage(hbm=kjt_size if topology.compute_device == "cuda" else 0, ddr=kjt_size if topology.compute_device in {"cpu", "mtia"} else 0)
    for device in topology.devices:
        device.storage -= kjt_storage
    return kjt_storage


def _reserve_storage_percentage(topology: Topology, percent: float) -> None:
    for device in topology.devices:
        device.storage.hbm = int((1 - percent) * device.storage.hbm)


class FixedPercentageStorageReservation(StorageReservation):
    def __init__(self, percentage: float) -> None:
        assert 0 <= percentage <= 1
        self._percentage = percentage
        self._last_reserved_topology: Optional[Topology] = None

    def reserve(self, topology, batch_size, module, sharders, constraints=None) -> Topology:
        reserved = copy.deepcopy(topology)
        _reserve_storage_percentage(reserved, self._percentage)
        self._last_reserved_topology = copy.deepcopy(reserved)
        return reserved

    @property
    def last_reserved_topology(self) -> Optional[Topology]:
        return self._last_reserved_topology


class HeuristicalStorageReservation(StorageReservation):
    """Reserve ``percentage`` of HBM for unknowns, plus the dense part (x6: weights, gradients, optimizer
    state, DDP buckets) and the input KJTs (x20: pipelined copies)."""

    def __init__(self, percentage: float, parameter_multiplier: float = 6.0, dense_tensor_estimate: Optional[int] = None) -> None:
        assert 0 <= percentage <= 1
        self._percentage = percentage
        self._parameter_multiplier = parameter_multiplier
        self._dense_tensor_estimate = dense_tensor_estimate
        self._dense_storage: Optional[Storage] = None
        self._kjt_storage: Optional[Storage] = None
        self._last_reserved_topology: Optional[Topology] = None

    def reserve(self, topology, batch_size, module, sharders, constraints=None) -> Topology:
        reserved = copy.deepcopy(topology)
        batch_inputs, shardable_modules = _get_batch_inputs_and_shardable_parameters(module, sharders, batch_size, constraints)
        _reserve_storage_percentage(reserved, self._percentage)
        self._dense_storage = _reserve_dense_storage(reserved, module, shardable_modules, self._parameter_multiplier, self._dense_tensor_estimate)
        self._kjt_storage = _reserve_kjt_storage(reserved, batch_size, batch_inputs, BIGINT_DTYPE, 20)
        if any(d.storage.hbm < 0 for d in reserved.devices) and reserved.compute_device == "cuda":
            negative = -min(d.storage.hbm for d in reserved.devices)
            raise PlannerError(
                error_type=PlannerErrorType.INSUFFICIENT_STORAGE,
                message=f"The storage reservation (dense {storage_repr_in_gb(self._dense_storage)}, kjt {storage_repr_in_gb(self._kjt_storage)}) exceeds the device memory by {negative} bytes.",
            )
        self._last_reserved_topology = copy.deepcopy(reserved)
        return reserved

    @property
    def last_reserved_topology(self) -> Optional[Topology]:
        return self._last_reserved_topology


class InferenceStorageReservation(StorageReservation):
    """Inference keeps weights only: dense part x1, no gradients or optimizer."""

    def __init__(self, percentage: float, dense_tensor_estimate: Optional[int] = None) -> None:
        assert 0 <= percentage <= 1
        self._percentage = percentage
        self._dense_tensor_estimate = dense_tensor_estimate
        self._dense_storage: Optional[Storage] = None
        self._kjt_storage: Optional[Storage] = None
        self._last_reserved_topology: Optional[Topology] = None

    def reserve(self, topology, batch_size, module, sharders, constraints=None) -> Topology:
        reserved = copy.deepcopy(topology)
        batch_inputs, shardable_modules = _get_batch_inputs_and_shardable_parameters(module, sharders, batch_size, constraints)
        _reserve_storage_percentage(reserved, self._percentage)
        self._dense_storage = _reserve_dense_storage(reserved, module, shardable_modules, 1, self._dense_tensor_estimate)
        self._kjt_storage = _reserve_kjt_storage(reserved, batch_size, batch_inputs, BIGINT_DTYPE, 1)
        self._last_reserved_topology = copy.deepcopy(reserved)
        return reserved

    @property
    def last_reserved_topology(self) -> Optional[Topology]:
        return self._last_reserved_topology
