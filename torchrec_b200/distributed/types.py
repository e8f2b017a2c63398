"""Core types of the sharding runtime.

API counterpart of ``torchrec/distributed/types.py`` (``ShardingType`` ``:118``,
``Awaitable``/``LazyAwaitable`` ``:324-463``, ``ParameterSharding`` ``:708``, ``ShardingPlan``
``:802``, ``ShardingEnv`` ``:855``, ``ShardedModule`` ``:989``, ``ModuleSharder`` ``:1152``).
``ShardedTensor``/``ShardMetadata`` come from ``torch.distributed._shard`` so that
checkpoints carry the same metadata as the reference's.
"""
from __future__ import annotations

import abc
import operator
from dataclasses import dataclass, field
from enum import Enum, unique
from typing import Any, Callable, Dict, Generic, Iterator, List, Optional, Tuple, Type, TypeVar, Union

import torch
import torch.distributed as dist
from torch import nn
from torch.autograd.profiler import record_function
from torch.distributed._shard.sharded_tensor import (  # noqa: F401
    Shard,
    ShardedTensor,
    ShardedTensorMetadata,
    TensorProperties,
)
from torch.distributed._shard.sharding_spec import (  # noqa: F401
    EnumerableShardingSpec,
    ShardingSpec,
    ShardMetadata,
)

from torchrec_b200.streamable import Multistreamable
from torchrec_b200.types import DataType


class ShardingType(Enum):
    DATA_PARALLEL = "data_parallel"
    TABLE_WISE = "table_wise"
    COLUMN_WISE = "column_wise"
    ROW_WISE = "row_wise"
    TABLE_ROW_WISE = "table_row_wise"
    TABLE_COLUMN_WISE = "table_column_wise"
    GRID_SHARD = "grid_shard"


class EmbeddingEvent(Enum):
    KJT_SPLITS_DIST = "splits_dist"
    KJT_TENSORS_DIST = "tensors_dist"
    LOOKUP = "lookup"
    OUTPUT_DIST = "output_dist"
    OUTPUT_DIST_WAIT = "output_dist_wait"


class PipelineType(Enum):
    NONE = "none"
    TRAIN_BASE = "train_base"
    TRAIN_SPARSE_DIST = "train_sparse_dist"
    TRAIN_PREFETCH_SPARSE_DIST = "train_prefetch_sparse_dist"


class ParameterStorage(Enum):
    HBM = "hbm"
    DDR = "ddr"
    SSD = "ssd"


class BoundsCheckMode(Enum):
    FATAL = 0
    WARNING = 1
    IGNORE = 2
    NONE = 3


class CacheAlgorithm(Enum):
    LRU = 0
    LFU = 1


@unique
class ComputeKernel(Enum):
    DEFAULT = "default"


# ---- quantized comms ---------------------------------------------------------------------
QuantizationContext = TypeVar("QuantizationContext")


class QuantizedCommCodec(Generic[QuantizationContext]):
    """Encode a tensor before a collective and decode it after."""

    def encode(self, input_tensor: torch.Tensor, ctx: Optional[QuantizationContext] = None) -> torch.Tensor:
        ...

    def decode(self, input_grad: torch.Tensor, ctx: Optional[QuantizationContext] = None) -> torch.Tensor:
        ...

    @property
    def quantized_dtype(self) -> torch.dtype:
        ...

    def calc_quantized_size(self, input_len: int, ctx: Optional[QuantizationContext] = None) -> int:
        ...

    def create_context(self) -> Optional[QuantizationContext]:
        ...

    def padded_size(self, input_tensor: torch.Tensor, dim_per_rank: List[int], my_rank: int, qcomm_ctx: QuantizationContext) -> Tuple[int, int]:
        return input_tensor.shape[-1], 0


class NoOpQuantizedCommCodec(QuantizedCommCodec):
    def encode(self, input_tensor, ctx=None):
        return input_tensor

    def decode(self, input_grad, ctx=None):
        return input_grad

    def quantized_dtype(self) -> torch.dtype:  # type: ignore[override]
        return torch.float

    def calc_quantized_size(self, input_len, ctx=None):
        return input_len

    def create_context(self):
        return None


@dataclass
class QuantizedCommCodecs:
    """Forward and backward codec of one collective."""

    forward: QuantizedCommCodec = field(default_factory=NoOpQuantizedCommCodec)
    backward: QuantizedCommCodec = field(default_factory=NoOpQuantizedCommCodec)


class CommOp(Enum):
    POOLED_EMBEDDINGS_ALL_TO_ALL = "pooled_embeddings_all_to_all"
    POOLED_EMBEDDINGS_REDUCE_SCATTER = "pooled_embeddings_reduce_scatter"
    SEQUENCE_EMBEDDINGS_ALL_TO_ALL = "sequence_embeddings_all_to_all"


# ---- awaitables ------------------------------------------------------------------------------
W = TypeVar("W")
M = TypeVar("M")


class Awaitable(abc.ABC, Generic[W]):
    """A result that may still be in flight; ``wait()`` returns it and runs the callbacks."""

    def __init__(self) -> None:
        self._callbacks: List[Callable[[W], W]] = []

    @abc.abstractmethod
    def _wait_impl(self) -> W:
        ...

    def wait(self) -> W:
        with record_function(f"## {self.__class__.__name__} wait() ##"):
            ret: W = self._wait_impl()
            for callback in self.callbacks:
                ret = callback(ret)
        return ret

    @property
    def callbacks(self) -> List[Callable[[W], W]]:
        return self._callbacks


class NoWait(Awaitable[W]):
    def __init__(self, obj: W) -> None:
        super().__init__()
        self._obj = obj

    def _wait_impl(self) -> W:
        return self._obj


class _LazyAwaitableMeta(abc.ABCMeta):
    pass


class LazyAwaitable(Awaitable[W], metaclass=_LazyAwaitableMeta):
    """An awaitable that waits by itself the first time its value is used.

    Attribute access, indexing, arithmetic and ``torch`` functions on the object first call
    ``wait()`` (once) and then act on the result, so model code can treat the output of a
    sharded module as the tensor / ``KeyedTensor`` / dict it will become.
    """

    def __init__(self) -> None:
        super().__init__()
        self._result: Optional[W] = None

    @staticmethod
    def _wait_async(obj: Any) -> Any:
        if isinstance(obj, LazyAwaitable):
            if obj._result is None:
                obj._result = obj.wait()
            return obj._result
        return obj

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        new_args = torch.fx.node.map_aggregate(args, LazyAwaitable._wait_async)
        new_kwargs = torch.fx.node.map_aggregate(kwargs, LazyAwaitable._wait_async)
        return func(*new_args, **new_kwargs)

    def __getattr__(self, name):
        if name in ("_result", "_callbacks") or name.startswith("__"):
            raise AttributeError(name)
        res = LazyAwaitable._wait_async(self)
        return getattr(res, name)


def _lazy_binop(op):
    def fwd(self, other):
        return op(LazyAwaitable._wait_async(self), LazyAwaitable._wait_async(other))

    def rev(self, other):
        return op(LazyAwaitable._wait_async(other), LazyAwaitable._wait_async(self))

    return fwd, rev


for _name, _op in (("add", operator.add), ("sub", operator.sub), ("mul", operator.mul), ("truediv", operator.truediv),
                   ("floordiv", operator.floordiv), ("mod", operator.mod), ("pow", operator.pow), ("matmul", operator.matmul)):
    _f, _r = _lazy_binop(_op)
    setattr(LazyAwaitable, f"__{_name}__", _f)
    setattr(LazyAwaitable, f"__r{_name}__", _r)
for _name, _op in (("lt", operator.lt), ("le", operator.le), ("gt", operator.gt), ("ge", operator.ge)):
    setattr(LazyAwaitable, f"__{_name}__", _lazy_binop(_op)[0])
setattr(LazyAwaitable, "__getitem__", lambda self, k: LazyAwaitable._wait_async(self)[k])
setattr(LazyAwaitable, "__len__", lambda self: len(LazyAwaitable._wait_async(self)))
setattr(LazyAwaitable, "__iter__", lambda self: iter(LazyAwaitable._wait_async(self)))
setattr(LazyAwaitable, "__neg__", lambda self: -LazyAwaitable._wait_async(self))
setattr(LazyAwaitable, "__abs__", lambda self: abs(LazyAwaitable._wait_async(self)))


class LazyNoWait(LazyAwaitable[W]):
    def __init__(self, obj: W) -> None:
        super().__init__()
        self._obj = obj

    def _wait_impl(self) -> W:
        return self._obj


class LazyGetItemMixin(Generic[W, M]):
    """``awaitable[key]`` without waiting: the lookup is deferred to a child awaitable."""

    def __getitem__(self, key):
        return GetItemLazyAwaitable(self, key)


class GetItemLazyAwaitable(LazyAwaitable[W]):
    def __init__(self, parent: LazyAwaitable, key) -> None:
        super().__init__()
        self._parent = parent
        self._key = key

    def _wait_impl(self) -> W:
        return LazyAwaitable._wait_async(self._parent)[self._key]


# ---- plan types --------------------------------------------------------------------------------
@dataclass
class CacheStatistics(abc.ABC):
    @property
    def expected_lookups(self) -> float:
        return 0.0

    def expected_miss_rate(self, clf: float) -> float:
        return 1.0

    @property
    def cacheability(self) -> float:
        return 0.0


@dataclass
class CacheParams:
    """Software-cache settings for tables kept partly outside HBM."""

    algorithm: Optional[CacheAlgorithm] = None
    load_factor: Optional[float] = None
    reserved_memory: Optional[float] = None
    precision: Optional[DataType] = None
    prefetch_pipeline: Optional[bool] = None
    stats: Optional[CacheStatistics] = None
    multipass_prefetch_config: Optional[Any] = None

    def __hash__(self) -> int:
        return hash((self.algorithm, self.load_factor, self.reserved_memory, self.precision, self.prefetch_pipeline))


@dataclass
class KeyValueParams:
    """Settings of key-value backed tables (SSD / parameter server)."""

    ssd_storage_directory: Optional[str] = None
    ssd_rocksdb_write_buffer_size: Optional[int] = None
    ssd_rocksdb_shards: Optional[int] = None
    ps_hosts: Optional[Tuple[Tuple[str, int], ...]] = None
    ps_client_thread_num: Optional[int] = None
    ps_max_key_per_request: Optional[int] = None
    ps_max_local_index_length: Optional[int] = None
    gather_ssd_cache_stats: Optional[bool] = None
    stats_reporter_config: Optional[Any] = None
    use_passed_in_path: bool = True
    l2_cache_size: Optional[int] = None
    max_l1_cache_size: Optional[int] = None
    enable_async_update: Optional[bool] = None
    bulk_init_chunk_size: Optional[int] = None
    lazy_bulk_init_enabled: Optional[bool] = None

    def __hash__(self) -> int:
        return hash((self.ssd_storage_directory, self.ssd_rocksdb_write_buffer_size, self.ssd_rocksdb_shards, self.ps_hosts,
                     self.ps_client_thread_num, self.ps_max_key_per_request, self.ps_max_local_index_length))


@dataclass
class ParameterSharding:
    """How one parameter (table) is sharded.

    ``ranks``: TABLE_WISE -> the owning rank; COLUMN_WISE -> rank of every column shard;
    TABLE_ROW_WISE -> first rank of the owning node; ROW_WISE / DATA_PARALLEL -> unused.
    """

    sharding_type: str
    compute_kernel: str
    ranks: Optional[List[int]] = None
    sharding_spec: Optional[ShardingSpec] = None
    cache_params: Optional[CacheParams] = None
    enforce_hbm: Optional[bool] = None
    stochastic_rounding: Optional[bool] = None
    bounds_check_mode: Optional[BoundsCheckMode] = None
    output_dtype: Optional[DataType] = None
    key_value_params: Optional[KeyValueParams] = None


class ModuleShardingPlan:
    pass


class EmbeddingModuleShardingPlan(ModuleShardingPlan, Dict[str, ParameterSharding]):
    """``{table name: ParameterSharding}`` of one embedding module."""

    def __str__(self) -> str:
        rows = []
        for name, ps in self.items():
            rows.append(f"{name}: {ps.sharding_type} / {ps.compute_kernel} / ranks={ps.ranks}")
            spec = ps.sharding_spec
            if spec is not None and hasattr(spec, "shards"):
                for s in spec.shards:
                    rows.append(f"    offsets={list(s.shard_offsets)} sizes={list(s.shard_sizes)} placement={s.placement}")
        return "\n".join(rows)


@dataclass
class ShardingPlan:
    """``{module path: ModuleShardingPlan}`` for a whole model."""

    plan: Dict[str, ModuleShardingPlan]

    def get_plan_for_module(self, module_path: str) -> Optional[ModuleShardingPlan]:
        return self.plan.get(module_path, None)

    def __str__(self) -> str:
        return "\n\n".join(f"module: {path}\n{plan}" for path, plan in self.plan.items())


# ---- environments --------------------------------------------------------------------------------
def _pg_device_type(pg: Optional[dist.ProcessGroup]) -> str:
    try:
        backend = dist.get_backend(pg)
    except Exception:
        return "cpu"
    return "cuda" if "nccl" in str(backend) else "cpu"


class ShardingEnv:
    """World size / rank / process group a module is sharded over.

    ``from_local`` builds an environment without a process group: one process driving
    several devices (inference).
    """

    def __init__(self, world_size: int, rank: int, pg: Optional[dist.ProcessGroup] = None, output_dtensor: bool = False) -> None:
        self.world_size = world_size
        self.rank = rank
        self.process_group: Optional[dist.ProcessGroup] = pg
        self.device_mesh = None
        self.output_dtensor: bool = output_dtensor

    @classmethod
    def from_process_group(cls, pg: dist.ProcessGroup) -> "ShardingEnv":
        return cls(dist.get_world_size(pg), dist.get_rank(pg), pg)

    @classmethod
    def from_local(cls, world_size: int, rank: int) -> "ShardingEnv":
        return cls(world_size, rank, None)


class ShardingEnv2D(ShardingEnv):
    """2D parallelism: shard inside ``sharding_pg``, replicate across the groups of ``global_pg``."""

    def __init__(self, sharding_pg, global_pg, device_mesh, node_group_size: Optional[int] = None, use_inter_host_allreduce: bool = False) -> None:
        assert device_mesh is None or device_mesh.ndim == 2, "DeviceMesh must be two dimensional!"
        self.world_size: int = dist.get_world_size(sharding_pg)
        self.global_world_size: int = dist.get_world_size(global_pg)
        self.rank: int = dist.get_rank(sharding_pg)
        self.global_rank: int = dist.get_rank(global_pg)
        self.process_group = global_pg
        self.sharding_pg = sharding_pg
        self.device_mesh = device_mesh
        self.node_group_size = node_group_size
        self.output_dtensor: bool = True
        self.use_inter_host_allreduce = use_inter_host_allreduce

    def num_sharding_groups(self) -> int:
        return self.global_world_size // self.world_size

    def remap_rank(self, rank: int, sharding_type: ShardingType) -> int:
        if sharding_type in (ShardingType.COLUMN_WISE, ShardingType.TABLE_WISE, ShardingType.GRID_SHARD):
            return rank % self.world_size if self.use_inter_host_allreduce else rank // self.num_sharding_groups()
        raise ValueError(f"Do not need 2D specific remapping logic for sharding type: {sharding_type}")


class NullShardingContext(Multistreamable):
    def record_stream(self, stream: torch.Stream) -> None:
        pass


class NullShardedModuleContext(NullShardingContext):
    """Context of a sharded module that carries nothing from its input dist to its output dist."""


Out = TypeVar("Out")
CompIn = TypeVar("CompIn")
DistOut = TypeVar("DistOut")
ShrdCtx = TypeVar("ShrdCtx", bound=Multistreamable)


class FeatureShardingMixIn:
    def feature_names(self) -> List[str]:
        raise NotImplementedError

    def feature_names_per_rank(self) -> List[List[str]]:
        raise NotImplementedError

    def features_per_rank(self) -> List[int]:
        raise NotImplementedError


class ModuleShardingMixIn:
    @property
    def shardings(self) -> Dict[str, FeatureShardingMixIn]:
        raise NotImplementedError


class ShardedModule(abc.ABC, nn.Module, Generic[CompIn, DistOut, Out, ShrdCtx], ModuleShardingMixIn):
    """A module whose forward is split into ``input_dist -> compute -> output_dist``.

    Train pipelines call the three stages separately to overlap the input all-to-all of the
    next batch with the current batch's dense compute.
    """

    _FORCE_STATE_DICT_LOAD = True

    def __init__(self, qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None) -> None:
        super().__init__()
        if qcomm_codecs_registry is None:
            qcomm_codecs_registry = {}
        self._qcomm_codecs_registry = qcomm_codecs_registry

    @abc.abstractmethod
    def create_context(self) -> ShrdCtx:
        ...

    @property
    def qcomm_codecs_registry(self) -> Optional[Dict[str, QuantizedCommCodecs]]:
        return self._qcomm_codecs_registry

    @abc.abstractmethod
    def input_dist(self, ctx: ShrdCtx, *input, **kwargs) -> Awaitable[Awaitable[CompIn]]:
        ...

    @abc.abstractmethod
    def compute(self, ctx: ShrdCtx, dist_input: CompIn) -> DistOut:
        ...

    @abc.abstractmethod
    def output_dist(self, ctx: ShrdCtx, output: DistOut) -> LazyAwaitable[Out]:
        ...

    def compute_and_output_dist(self, ctx: ShrdCtx, input: CompIn) -> LazyAwaitable[Out]:
        output = self.compute(ctx, input)
        return self.output_dist(ctx, output)

    def forward(self, *input, **kwargs) -> LazyAwaitable[Out]:
        ctx = self.create_context()
        dist_input = self.input_dist(ctx, *input, **kwargs).wait().wait()
        return self.compute_and_output_dist(ctx, dist_input)

    def sharded_parameter_names(self, prefix: str = "") -> Iterator[str]:
        for key, _ in self.named_parameters(prefix):
            yield key

    @property
    @abc.abstractmethod
    def unsharded_module_type(self) -> Type[nn.Module]:
        ...


def get_tensor_size_bytes(t: torch.Tensor) -> int:
    b = t.numel() * t.element_size()
    return b


class ModuleSharder(abc.ABC, Generic[M]):
    """Turns an unsharded module of type ``module_type`` into its sharded counterpart."""

    def __init__(self, qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None) -> None:
        self._qcomm_codecs_registry = qcomm_codecs_registry

    @abc.abstractmethod
    def shard(self, module: M, params: EmbeddingModuleShardingPlan, env: ShardingEnv, device: Optional[torch.device] = None, module_fqn: Optional[str] = None) -> ShardedModule:
        ...

    @property
    @abc.abstractmethod
    def module_type(self) -> Type[M]:
        ...

    @property
    def qcomm_codecs_registry(self) -> Optional[Dict[str, QuantizedCommCodecs]]:
        return self._qcomm_codecs_registry

    def shardable_parameters(self, module: M) -> Dict[str, nn.Parameter]:
        return dict(module.named_parameters())

    def sharding_types(self, compute_device_type: str) -> List[str]:
        return [ShardingType.DATA_PARALLEL.value]

    def compute_kernels(self, sharding_type: str, compute_device_type: str) -> List[str]:
        return [ComputeKernel.DEFAULT.value]

    def storage_usage(self, tensor: torch.Tensor, compute_device_type: str, compute_kernel: str) -> Dict[str, int]:
        assert compute_device_type in {"cuda", "cpu", "mtia"}
        storage_map = {"cuda": ParameterStorage.HBM, "cpu": ParameterStorage.DDR, "mtia": ParameterStorage.DDR}
        return {storage_map[compute_device_type].value: get_tensor_size_bytes(tensor)}


class ShardingPlanner(abc.ABC):
    @abc.abstractmethod
    def plan(self, module: nn.Module, sharders: List[ModuleSharder]) -> ShardingPlan:
        ...

    @abc.abstractmethod
    def collective_plan(self, module: nn.Module, sharders: List[ModuleSharder], pg: Optional[dist.ProcessGroup]) -> ShardingPlan:
        ...


class ObjectPoolShardingType(Enum):
    ROW_WISE = "row_wise"
    REPLICATED_ROW_WISE = "replicated_row_wise"


@dataclass
class ObjectPoolShardingPlan(ModuleShardingPlan):
    sharding_type: ObjectPoolShardingType
    inference: bool = False


@dataclass
class DMPCollectionConfig:
    module: Type[nn.Module]
    plan: "ShardingPlan"
    sharding_group_size: int
    node_group_size: Optional[int] = None
    use_inter_host_allreduce: bool = False


class DMPCollectionContext(DMPCollectionConfig):
    def __init__(self, module, plan, sharding_group_size, node_group_size=None, use_inter_host_allreduce=False) -> None:
        super().__init__(module, plan, sharding_group_size, node_group_size, use_inter_host_allreduce)
        self.device_mesh = None
        self.sharding_pg = None
        self.replica_pg = None
        self.modules_to_sync: List[Tuple[nn.Module, nn.Module]] = []
        self.sharded_module: Optional[Type[nn.Module]] = None


def rank_device(device_type: str, rank: int) -> torch.device:
    """The device of ``rank`` in a job with one device per rank (the host has a single device)."""
    return torch.device("cpu") if device_type == "cpu" else torch.device(f"{device_type}:{rank}")


@dataclass
class ShardingBucketMetadata:
    """Bucket layout of a row-wise table that is sharded on bucket boundaries: how many buckets every shard holds, the index of
    every shard's first bucket, and the rows per bucket."""

    num_buckets_per_shard: List[int]
    bucket_offsets_per_shard: List[int]
    bucket_size: int
