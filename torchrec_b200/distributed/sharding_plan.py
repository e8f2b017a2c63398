"""Helpers to write sharding plans by hand.

Counterpart of ``torchrec/distributed/sharding_plan.py:48-966``:
``calculate_shard_sizes_and_offsets`` defines the shard geometry of every sharding type
(row-wise uses ``ceil(rows / W)`` blocks so a trailing rank may own fewer or zero rows;
column-wise splits ``D`` into equal blocks that divide it and are multiples of 4), and the
``table_wise() / row_wise() / column_wise() / table_row_wise() / grid_shard() /
data_parallel()`` generators feed ``construct_module_sharding_plan``.
"""
from __future__ import annotations

import math
import warnings
from typing import Callable, Dict, List, Optional, Tuple, Type, Union

import torch
from torch import nn

from torchrec_b200.distributed.embedding_types import EmbeddingComputeKernel
from torchrec_b200.distributed.types import (
    EmbeddingModuleShardingPlan,
    EnumerableShardingSpec,
    ModuleSharder,
    ParameterSharding,
    ShardingType,
    ShardMetadata,
)

MIN_CW_DIM: int = 128


def get_default_sharders() -> List[ModuleSharder[nn.Module]]:
    """One sharder per shardable module type the framework knows."""
    from torchrec_b200.distributed.embeddingbag import EmbeddingBagCollectionSharder

    sharders: List[ModuleSharder[nn.Module]] = [EmbeddingBagCollectionSharder()]
    for modname, clsname in (
        ("torchrec_b200.distributed.embedding", "EmbeddingCollectionSharder"),
        ("torchrec_b200.distributed.fp_embeddingbag", "FeatureProcessedEmbeddingBagCollectionSharder"),
        ("torchrec_b200.distributed.fused_embeddingbag", "FusedEmbeddingBagCollectionSharder"),
        ("torchrec_b200.distributed.fused_embeddingbag", "FusedEmbeddingCollectionSharder"),
        ("torchrec_b200.distributed.quant_embeddingbag", "QuantEmbeddingBagCollectionSharder"),
        ("torchrec_b200.distributed.quant_embedding", "QuantEmbeddingCollectionSharder"),
        ("torchrec_b200.distributed.mc_embeddingbag", "ManagedCollisionEmbeddingBagCollectionSharder"),
        ("torchrec_b200.distributed.mc_embedding", "ManagedCollisionEmbeddingCollectionSharder"),
        ("torchrec_b200.distributed.itep_embeddingbag", "ITEPEmbeddingBagCollectionSharder"),
        ("torchrec_b200.distributed.itep_embeddingbag", "ITEPEmbeddingCollectionSharder"),
    ):
        try:
            mod = __import__(modname, fromlist=[clsname])
            sharders.append(getattr(mod, clsname)())
        except ImportError:
            pass
    return sharders


def get_module_to_default_sharders() -> Dict[Type[nn.Module], ModuleSharder[nn.Module]]:
    return {sharder.module_type: sharder for sharder in get_default_sharders()}


def placement(compute_device: str, rank: int, local_size: int) -> str:
    param_device = compute_device
    if compute_device in {"cuda", "mtia"}:
        param_device = f"{compute_device}:{rank % local_size}"
    return f"rank:{rank}/{param_device}"


def placement_helper(device_type: str, index: int = 0, rank: int = 0) -> str:
    """The placement string of a shard: ``rank:<rank>/<device>:<index>``; host memory is always written as rank 0's."""
    if device_type == "cpu":
        return f"rank:0/{device_type}"
    return f"rank:{rank}/{device_type}:{index}"


def _rw(hash_size: int, num_devices: int, columns: int, num_buckets: Optional[int] = None):
    shard_sizes: List[List[int]] = []
    if num_buckets:
        assert hash_size % num_buckets == 0, "hash_size must be divisible by num_buckets"
        bucket_size = hash_size // num_buckets
        shard_buckets = num_buckets // num_devices
        extra = num_buckets % num_devices
        for rank in range(num_devices):
            shard_sizes.append([bucket_size * (shard_buckets + (1 if rank < extra else 0)), columns])
    else:
        block_size = math.ceil(hash_size / num_devices)
        last_rank = hash_size // block_size
        last_block_size = hash_size - block_size * last_rank
        for rank in range(num_devices):
            local_row = block_size if rank < last_rank else (last_block_size if rank == last_rank else 0)
            shard_sizes.append([local_row, columns])
    shard_offsets = [[0, 0]]
    for i in range(num_devices - 1):
        shard_offsets.append([shard_sizes[i][0] + shard_offsets[i][0], 0])
    return shard_sizes, shard_offsets


def _uneven_rw(hash_size: int, num_devices: int, columns: int, device_memory_sizes: List[int], num_buckets: Optional[int] = None):
    assert num_devices == len(device_memory_sizes), "must provide all the memory size"
    total = sum(device_memory_sizes)
    if num_buckets is None:
        num_buckets, bucket_size = hash_size, 1
    else:
        assert hash_size % num_buckets == 0
        bucket_size = hash_size // num_buckets
    shard_sizes, done = [], 0
    for rank in range(num_devices):
        if rank < num_devices - 1:
            local = int(num_buckets * (device_memory_sizes[rank] / total)) * bucket_size
            done += local
        else:
            local = hash_size - done
        shard_sizes.append([local, columns])
    shard_offsets = [[0, 0]]
    for i in range(num_devices - 1):
        shard_offsets.append([shard_sizes[i][0] + shard_offsets[i][0], 0])
    return shard_sizes, shard_offsets


def _find_base_dim(lower_bound: int, dim: int) -> int:
    for i in range(lower_bound, dim):
        if dim % i == 0 and i % 4 == 0:
            return i
    return dim


def _get_block_size_for_cw_shard(columns: int, column_wise_shard_dim: Optional[int]) -> int:
    block_size = min(_find_base_dim(column_wise_shard_dim or MIN_CW_DIM, columns), columns)
    if columns % block_size != 0:
        warnings.warn(
            f"Dim of {columns} cannot be evenly divided with column wise shard dim {column_wise_shard_dim}, "
            f"overriding block_size to embedding_dim={columns}", UserWarning, stacklevel=2,
        )
        block_size = columns
    return block_size


def _cw(columns: int, rows: int, col_wise_shard_dim: Optional[int] = None):
    block = _get_block_size_for_cw_shard(columns, col_wise_shard_dim)
    n = columns // block
    return [[rows, block]] * n, [[0, block * r] for r in range(n)]


def _grid(hash_size: int, num_device: int, columns: int, col_wise_shard_dim: Optional[int] = None):
    row_sizes, row_offsets = _rw(hash_size, num_device, columns)
    block = _get_block_size_for_cw_shard(columns, col_wise_shard_dim)
    sizes, offsets = [], []
    for node in range(columns // block):
        for rs, ro in zip(row_sizes, row_offsets):
            sizes.append([rs[0], block])
            offsets.append([ro[0], block * node])
    return sizes, offsets


def calculate_shard_sizes_and_offsets(
    tensor: torch.Tensor,
    world_size: int,
    local_world_size: int,
    sharding_type: str,
    col_wise_shard_dim: Optional[int] = None,
    device_memory_sizes: Optional[List[int]] = None,
    num_buckets: Optional[int] = None,
) -> Tuple[List[List[int]], List[List[int]]]:
    """Shard sizes and offsets of ``tensor [rows, cols]`` for ``sharding_type``."""
    rows, columns = tensor.shape
    if sharding_type == ShardingType.DATA_PARALLEL.value:
        return [[rows, columns]] * world_size, [[0, 0]] * world_size
    if sharding_type == ShardingType.TABLE_WISE.value:
        return [[rows, columns]], [[0, 0]]
    if sharding_type == ShardingType.ROW_WISE.value:
        if device_memory_sizes:
            return _uneven_rw(rows, world_size, columns, device_memory_sizes, num_buckets)
        return _rw(rows, world_size, columns, num_buckets)
    if sharding_type == ShardingType.TABLE_ROW_WISE.value:
        return _rw(rows, local_world_size, columns)
    if sharding_type in (ShardingType.COLUMN_WISE.value, ShardingType.TABLE_COLUMN_WISE.value):
        return _cw(columns, rows, col_wise_shard_dim)
    if sharding_type == ShardingType.GRID_SHARD.value:
        return _grid(rows, local_world_size, columns, col_wise_shard_dim)
    raise ValueError(f"Unrecognized or unsupported sharding type provided: {sharding_type}")


def _get_parameter_size_offsets(param, sharding_type: ShardingType, local_size: int, world_size: int, col_wise_shard_dim: Optional[int] = None):
    sizes, offsets = calculate_shard_sizes_and_offsets(param, world_size, local_size, sharding_type.value, col_wise_shard_dim)
    return list(zip(sizes, offsets))


def _get_compute_kernel(sharder, param, sharding_type: str, device_type: str) -> str:
    if sharding_type == ShardingType.DATA_PARALLEL.value:
        return EmbeddingComputeKernel.DENSE.value
    if hasattr(param, "_in_backward_optimizers") or getattr(param, "_optimizer_classes", None):
        return EmbeddingComputeKernel.FUSED.value
    return EmbeddingComputeKernel.DENSE.value


def _get_parameter_sharding(
    param, sharding_type: str, size_offset_ranks, local_size: int, device_type: str, sharder,
    placements: Optional[List[str]] = None, compute_kernel: Optional[str] = None,
) -> ParameterSharding:
    spec = None
    if sharding_type != ShardingType.DATA_PARALLEL.value:
        spec = EnumerableShardingSpec(
            [
                ShardMetadata(
                    shard_sizes=size, shard_offsets=offset,
                    placement=(placement(device_type, rank, local_size) if not dp else dp),
                )
                for (size, offset, rank), dp in zip(size_offset_ranks, placements if placements else [None] * len(size_offset_ranks))
            ]
        )
    return ParameterSharding(
        sharding_spec=spec,
        sharding_type=sharding_type,
        compute_kernel=compute_kernel if compute_kernel else _get_compute_kernel(sharder, param, sharding_type, device_type),
        ranks=[rank for (_, _, rank) in size_offset_ranks],
    )


ParameterShardingGenerator = Callable[[nn.Parameter, int, int, str, ModuleSharder[nn.Module]], ParameterSharding]


def data_parallel() -> ParameterShardingGenerator:
    """Replicate the table on every rank (dense gradient, all-reduced)."""

    def gen(param, local_size, world_size, device_type, sharder):
        so = _get_parameter_size_offsets(param, ShardingType.DATA_PARALLEL, local_size, world_size)
        so_ranks = [(so[i][0], so[i][1], i) for i in range(world_size)]
        return _get_parameter_sharding(param, ShardingType.DATA_PARALLEL.value, so_ranks, local_size, device_type, sharder)

    return gen


def table_wise(rank: int, device: Optional[str] = None, compute_kernel: Optional[str] = None) -> ParameterShardingGenerator:
    """Place the whole table on ``rank``."""

    def gen(param, local_size, world_size, device_type, sharder):
        so = _get_parameter_size_offsets(param, ShardingType.TABLE_WISE, local_size, world_size)
        assert len(so) == 1
        so_ranks = [(so[0][0], so[0][1], rank)]
        return _get_parameter_sharding(
            param, ShardingType.TABLE_WISE.value, so_ranks, local_size, device or device_type, sharder,
            compute_kernel=compute_kernel,
        )

    return gen


def row_wise(
    sizes_placement: Optional[Tuple[List[int], Union[str, List[str]]]] = None,
    compute_kernel: Optional[str] = None,
) -> ParameterShardingGenerator:
    """Split rows over all ranks; ``sizes_placement=([rows per shard], device or devices)`` gives uneven splits."""
    if sizes_placement is not None and isinstance(sizes_placement[1], list):
        assert len(sizes_placement[0]) == len(sizes_placement[1]), "sizes_placement and device per placement (in case of sharding across HBM and CPU host) must have the same length"

    def gen(param, local_size, world_size, device_type, sharder):
        if sizes_placement is None:
            so = _get_parameter_size_offsets(param, ShardingType.ROW_WISE, local_size, world_size)
        else:
            so, off = [], 0
            for s in sizes_placement[0]:
                so.append(([s, param.shape[1]], [off, 0]))
                off += s
        assert len(so) <= world_size
        so_ranks = [(s, o, r) for r, (s, o) in enumerate(so)]
        placements = None
        ck = compute_kernel
        dt = device_type
        if sizes_placement is not None:
            if isinstance(sizes_placement[1], list):
                placements = [placement(d, r, local_size) for r, d in enumerate(sizes_placement[1])]
            else:
                dt = sizes_placement[1]
            if ck is None:
                ck = EmbeddingComputeKernel.QUANT.value
        return _get_parameter_sharding(param, ShardingType.ROW_WISE.value, so_ranks, local_size, dt, sharder, placements=placements, compute_kernel=ck)

    return gen


def column_wise(
    ranks: Optional[List[int]] = None, size_per_rank: Optional[List[int]] = None, compute_kernel: Optional[str] = None,
) -> ParameterShardingGenerator:
    """Split columns evenly over ``ranks`` (or into the widths ``size_per_rank``)."""
    if ranks is None and size_per_rank is None:
        raise ValueError("Either ranks or size_per_rank must be specified")

    def gen(param, local_size, world_size, device_type, sharder):
        rr = ranks if ranks is not None else list(range(len(size_per_rank)))
        if size_per_rank is None:
            if param.shape[1] % len(rr) != 0:
                raise ValueError(f"column dim of {param.shape[1]} cannot be evenly divided across {rr}")
            shard_dim = param.shape[1] // len(rr)
            so = _get_parameter_size_offsets(param, ShardingType.COLUMN_WISE, local_size, world_size, col_wise_shard_dim=shard_dim)
        else:
            if sum(size_per_rank) != param.shape[1]:
                raise ValueError(f"sum of size_per_rank {size_per_rank} must match the column dim {param.shape[1]}")
            so, off = [], 0
            for s in size_per_rank:
                so.append(([param.shape[0], s], [0, off]))
                off += s
        so_ranks = [(s, o, r) for (s, o), r in zip(so, rr)]
        return _get_parameter_sharding(param, ShardingType.COLUMN_WISE.value, so_ranks, local_size, device_type, sharder, compute_kernel=compute_kernel)

    return gen


def table_row_wise(host_index: int, compute_kernel: Optional[str] = None) -> ParameterShardingGenerator:
    """Place the table on node ``host_index`` and split its rows over that node's ranks."""

    def gen(param, local_size, world_size, device_type, sharder):
        so = _get_parameter_size_offsets(param, ShardingType.TABLE_ROW_WISE, local_size, world_size)
        first = host_index * local_size
        so_ranks = [(s, o, first + i) for i, (s, o) in enumerate(so)]
        return _get_parameter_sharding(param, ShardingType.TABLE_ROW_WISE.value, so_ranks, local_size, device_type, sharder, compute_kernel=compute_kernel)

    return gen


def grid_shard(host_indexes: List[int], compute_kernel: Optional[str] = None) -> ParameterShardingGenerator:
    """Column shards across ``host_indexes``, each split row-wise over its node."""

    def gen(param, local_size, world_size, device_type, sharder):
        so = _get_parameter_size_offsets(
            param, ShardingType.GRID_SHARD, local_size, world_size, col_wise_shard_dim=param.shape[1] // len(host_indexes),
        )
        size_offset_ranks = []
        for i, (s, o) in enumerate(so):
            h = host_indexes[i // local_size]
            size_offset_ranks.append((s, o, h * local_size + i % local_size))
        return _get_parameter_sharding(param, ShardingType.GRID_SHARD.value, size_offset_ranks, local_size, device_type, sharder, compute_kernel=compute_kernel)

    return gen


def get_sharding_constructor_from_type(sharding_type: ShardingType) -> Callable[..., ParameterShardingGenerator]:
    return {
        ShardingType.TABLE_WISE: table_wise, ShardingType.ROW_WISE: row_wise, ShardingType.COLUMN_WISE: column_wise,
        ShardingType.TABLE_ROW_WISE: table_row_wise, ShardingType.GRID_SHARD: grid_shard, ShardingType.DATA_PARALLEL: data_parallel,
    }[sharding_type]


def apply_to_all(module: nn.Module, parameter_sharding_generator: ParameterShardingGenerator, sharder=None) -> Dict[str, ParameterShardingGenerator]:
    if sharder is None:
        sharder = get_module_to_default_sharders().get(type(module), None)
    assert sharder is not None, f"Could not find a valid sharder type for {type(module)}"
    return {name: parameter_sharding_generator for name in sharder.shardable_parameters(module).keys()}


def construct_module_sharding_plan(
    module: nn.Module,
    per_param_sharding: Dict[str, ParameterShardingGenerator],
    sharder: Optional[ModuleSharder[nn.Module]] = None,
    local_size: Optional[int] = None,
    world_size: Optional[int] = None,
    device_type: Optional[str] = None,
) -> EmbeddingModuleShardingPlan:
    """Build a module plan from ``{table name: generator}``."""
    import torch.distributed as dist
    from torchrec_b200.distributed.comm import get_local_size

    if device_type is None:
        device_type = "cuda" if torch.cuda.is_available() else "cpu"
    if sharder is None:
        sharder = get_module_to_default_sharders().get(type(module), None)
    assert sharder is not None, f"Could not find a valid sharder type for {type(module)}"
    assert isinstance(module, sharder.module_type), f"Incorrect sharder for module type {type(module)}"
    shardable = sharder.shardable_parameters(module)
    assert shardable.keys() == per_param_sharding.keys(), "per_param_sharding_config doesn't match the shardable parameters of the module"
    if world_size is None:
        world_size = dist.get_world_size()
    if local_size is None:
        local_size = get_local_size(world_size)
    plan = EmbeddingModuleShardingPlan()
    for name, gen in per_param_sharding.items():
        plan[name] = gen(shardable[name], local_size, world_size, device_type, sharder)
    return plan
