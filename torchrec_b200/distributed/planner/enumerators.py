"""Search-space enumeration: every (table x sharding type x compute kernel) allowed by the sharder
and the user's constraints becomes a ``ShardingOption`` with shard sizes/offsets and estimates.
Counterpart of ``torchrec/distributed/planner/enumerators.py``.
"""
from __future__ import annotations

import copy
import logging
from typing import Dict, List, Optional, Set, Tuple, Union

from torch import nn

from torchrec_b200.distributed.embedding_types import EmbeddingComputeKernel
from torchrec_b200.distributed.planner.constants import BATCH_SIZE, POOLING_FACTOR
from torchrec_b200.distributed.planner.types import (
    Enumerator,
    ParameterConstraints,
    PartitionByType,
    Shard,
    ShardEstimator,
    ShardingOption,
    Topology,
)
from torchrec_b200.distributed.planner.utils import sharder_name
from torchrec_b200.distributed.sharding_plan import calculate_shard_sizes_and_offsets
from torchrec_b200.distributed.types import BoundsCheckMode, CacheParams, KeyValueParams, ModuleSharder, ShardingType

logger: logging.Logger = logging.getLogger(__name__)

GUARDED_COMPUTE_KERNELS: Set[EmbeddingComputeKernel] = {EmbeddingComputeKernel.KEY_VALUE, EmbeddingComputeKernel.SSD_VIRTUAL_TABLE, EmbeddingComputeKernel.DRAM_VIRTUAL_TABLE}


def get_partition_by_type(sharding_type: str) -> str:
    """Granularity at which the partitioner must place a sharding type."""
    device = {ShardingType.TABLE_WISE.value, ShardingType.COLUMN_WISE.value}
    host = {ShardingType.TABLE_ROW_WISE.value, ShardingType.TABLE_COLUMN_WISE.value}
    uniform = {ShardingType.ROW_WISE.value, ShardingType.DATA_PARALLEL.value}
    multi_host = {ShardingType.GRID_SHARD.value}
    if sharding_type in device:
        return PartitionByType.DEVICE.value
    if sharding_type in host:
        return PartitionByType.HOST.value
    if sharding_type in multi_host:
        return PartitionByType.MULTI_HOST.value
    if sharding_type in uniform:
        return PartitionByType.UNIFORM.value
    raise ValueError(f"Unrecognized or unsupported sharding type provided: {sharding_type}")


class EmbeddingEnumerator(Enumerator):
    def __init__(self, topology: Topology, batch_size: int = BATCH_SIZE, constraints: Optional[Dict[str, ParameterConstraints]] = None,
                 estimator: Optional[Union[ShardEstimator, List[ShardEstimator]]] = None, use_exact_enumerate_order: Optional[bool] = False) -> None:
        self._compute_device: str = topology.compute_device
        self._world_size: int = topology.world_size
        self._local_world_size: int = topology.local_world_size
        self._batch_size: int = batch_size
        self._constraints = constraints
        self._sharder_map: Dict[str, ModuleSharder[nn.Module]] = {}
        self._use_exact_enumerate_order = bool(use_exact_enumerate_order)
        self.last_stored_search_space: Optional[List[ShardingOption]] = None
        if estimator:
            self._estimators: List[ShardEstimator] = [estimator] if not isinstance(estimator, list) else estimator
        else:
            from torchrec_b200.distributed.planner.shard_estimators import EmbeddingPerfEstimator, EmbeddingStorageEstimator

            self._estimators = [EmbeddingPerfEstimator(topology=topology, constraints=constraints), EmbeddingStorageEstimator(topology=topology, constraints=constraints)]

    def enumerate(self, module: nn.Module, sharders: List[ModuleSharder[nn.Module]]) -> List[ShardingOption]:
        self._sharder_map = {sharder_name(s.module_type): s for s in sharders}
        sharding_options: List[ShardingOption] = []
        named_modules = list(module.named_modules())
        for child_path, child_module in named_modules:
            key = sharder_name(type(child_module))
            sharder = self._sharder_map.get(key, None)
            if not sharder:
                continue
            for name, param in sharder.shardable_parameters(child_module).items():
                (input_lengths, col_wise_shard_dim, cache_params, enforce_hbm, stochastic_rounding, bounds_check_mode,
                 feature_names, output_dtype, device_group, key_value_params) = _extract_constraints_for_param(self._constraints, name)
                if device_group and device_group != self._compute_device:
                    continue
                sharding_options_per_table: List[ShardingOption] = []
                for sharding_type in self._filter_sharding_types(name, sharder.sharding_types(self._compute_device)):
                    for compute_kernel in self._filter_compute_kernels(name, sharder.compute_kernels(sharding_type, self._compute_device), sharding_type):
                        shard_sizes, shard_offsets = calculate_shard_sizes_and_offsets(
                            tensor=param, world_size=self._world_size, local_world_size=self._local_world_size,
                            sharding_type=sharding_type, col_wise_shard_dim=col_wise_shard_dim,
                        )
                        dependency = None
                        if isinstance(child_module, _EmbeddingTowerTypes):
                            dependency = child_path
                        sharding_options_per_table.append(
                            ShardingOption(
                                name=name, tensor=param, module=(child_path, child_module), input_lengths=input_lengths,
                                batch_size=self._batch_size, compute_kernel=compute_kernel, sharding_type=sharding_type,
                                partition_by=get_partition_by_type(sharding_type),
                                shards=[Shard(size=size, offset=offset) for size, offset in zip(shard_sizes, shard_offsets)],
                                cache_params=cache_params, enforce_hbm=enforce_hbm, stochastic_rounding=stochastic_rounding,
                                bounds_check_mode=bounds_check_mode, dependency=dependency, feature_names=feature_names,
                                output_dtype=output_dtype, key_value_params=key_value_params,
                            )
                        )
                if not sharding_options_per_table:
                    raise RuntimeError(
                        f"No available sharding type and compute kernel combination for {name} after applying user provided constraints"
                    )
                sharding_options.extend(sharding_options_per_table)
        self.populate_estimates(sharding_options)
        self.last_stored_search_space = copy.deepcopy(sharding_options)
        return sharding_options

    @property
    def last_stored_search_space(self) -> Optional[List[ShardingOption]]:
        return self._last_stored_search_space

    @last_stored_search_space.setter
    def last_stored_search_space(self, v) -> None:
        self._last_stored_search_space = v

    def populate_estimates(self, sharding_options: List[ShardingOption]) -> None:
        for estimator in self._estimators:
            estimator.estimate(sharding_options, self._sharder_map)

    def _filter_sharding_types(self, name: str, allowed_sharding_types: List[str]) -> List[str]:
        # grid sharding is only considered when asked for explicitly
        filtered = [t for t in allowed_sharding_types if t != ShardingType.GRID_SHARD.value]
        if not self._constraints or not self._constraints.get(name):
            return filtered
        constraints = self._constraints[name]
        if not constraints.sharding_types:
            return filtered
        constrained = constraints.sharding_types
        out = list(set(constrained) & set(allowed_sharding_types))
        if self._use_exact_enumerate_order:
            out = [t for t in constrained if t in allowed_sharding_types]
        if not out:
            logger.warning(f"No available sharding types after applying user provided constraints for {name}. Constrained: {constrained}, allowed: {allowed_sharding_types}")
        return sorted(out) if not self._use_exact_enumerate_order else out

    def _filter_compute_kernels(self, name: str, allowed_compute_kernels: List[str], sharding_type: str) -> List[str]:
        constrained = [k.value for k in EmbeddingComputeKernel if k not in GUARDED_COMPUTE_KERNELS]
        if self._constraints and self._constraints.get(name) and self._constraints[name].compute_kernels:
            constrained = self._constraints[name].compute_kernels
        filtered = list(set(constrained) & set(allowed_compute_kernels))
        if EmbeddingComputeKernel.DENSE.value in filtered and EmbeddingComputeKernel.FUSED.value in filtered:
            filtered.remove(EmbeddingComputeKernel.DENSE.value)
        if not filtered:
            logger.warning(f"No available compute kernels after applying user provided constraints for {name}")
        return sorted(filtered)


class _NoTower:
    pass


try:
    from torchrec_b200.modules.embedding_tower import EmbeddingTower, EmbeddingTowerCollection

    _EmbeddingTowerTypes: Tuple[type, ...] = (EmbeddingTower, EmbeddingTowerCollection)
except ImportError:
    _EmbeddingTowerTypes = (_NoTower,)


def _extract_constraints_for_param(constraints: Optional[Dict[str, ParameterConstraints]], name: str):
    input_lengths = [POOLING_FACTOR]
    col_wise_shard_dim = cache_params = enforce_hbm = stochastic_rounding = bounds_check_mode = None
    feature_names = output_dtype = device_group = key_value_params = None
    if constraints and constraints.get(name):
        c = constraints[name]
        input_lengths = c.pooling_factors
        col_wise_shard_dim = c.min_partition
        cache_params = c.cache_params
        enforce_hbm = c.enforce_hbm
        stochastic_rounding = c.stochastic_rounding
        bounds_check_mode = c.bounds_check_mode
        feature_names = c.feature_names
        output_dtype = c.output_dtype
        device_group = c.device_group
        key_value_params = c.key_value_params
    return (input_lengths, col_wise_shard_dim, cache_params, enforce_hbm, stochastic_rounding, bounds_check_mode,
            feature_names, output_dtype, device_group, key_value_params)
