"""Types shared by the sharded embedding modules (cf. ``torchrec/distributed/embedding_types.py``)."""
from __future__ import annotations

import abc
import copy
from dataclasses import dataclass, field
from enum import Enum, unique
from typing import Any, Dict, Generic, Iterator, List, Optional, Tuple, TypeVar, Union

import torch
from torch import fx, nn

from torchrec_b200.distributed.types import (
    BoundsCheckMode,
    CacheParams,
    EnumerableShardingSpec,
    KeyValueParams,
    ModuleSharder,
    ParameterStorage,
    QuantizedCommCodecs,
    ShardedModule,
    ShardedTensorMetadata,
    ShardingType,
    ShardMetadata,
    get_tensor_size_bytes,
)
from torchrec_b200.modules.embedding_configs import DataType, EmbeddingTableConfig, PoolingType
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor
from torchrec_b200.streamable import Multistreamable


@unique
class OptimType(Enum):
    SGD = "SGD"
    LARS_SGD = "LARS_SGD"
    LAMB = "LAMB"
    PARTIAL_ROWWISE_LAMB = "PARTIAL_ROWWISE_LAMB"
    ADAM = "ADAM"
    PARTIAL_ROWWISE_ADAM = "PARTIAL_ROWWISE_ADAM"
    ADAGRAD = "ADAGRAD"
    ROWWISE_ADAGRAD = "ROWWISE_ADAGRAD"
    SHAMPOO = "SHAMPOO"
    SHAMPOO_V2 = "SHAMPOO_V2"
    LION = "LION"
    ADAMW = "ADAMW"
    SHAMPOO_V2_MRS = "SHAMPOO_V2_MRS"
    SHAMPOO_MRS = "SHAMPOO_MRS"


@unique
class EmbeddingComputeKernel(Enum):
    DENSE = "dense"
    FUSED = "fused"
    FUSED_UVM = "fused_uvm"
    FUSED_UVM_CACHING = "fused_uvm_caching"
    QUANT = "quant"
    QUANT_UVM = "quant_uvm"
    QUANT_UVM_CACHING = "quant_uvm_caching"
    KEY_VALUE = "key_value"
    CUSTOMIZED_KERNEL = "customized_kernel"
    SSD_VIRTUAL_TABLE = "ssd_virtual_table"
    DRAM_VIRTUAL_TABLE = "dram_virtual_table"


def compute_kernel_to_embedding_location(compute_kernel: EmbeddingComputeKernel) -> str:
    if compute_kernel in (EmbeddingComputeKernel.DENSE, EmbeddingComputeKernel.FUSED, EmbeddingComputeKernel.QUANT):
        return "device"
    if compute_kernel in (EmbeddingComputeKernel.FUSED_UVM, EmbeddingComputeKernel.QUANT_UVM):
        return "managed"
    if compute_kernel in (EmbeddingComputeKernel.FUSED_UVM_CACHING, EmbeddingComputeKernel.QUANT_UVM_CACHING):
        return "managed_caching"
    return "host"


@dataclass
class DTensorMetadata:
    """What is needed to present a table's local shards as a ``DTensor``: the device mesh, the placements on it, and the global
    size and stride."""

    mesh: Optional[Any] = None
    placements: Optional[Tuple[Any, ...]] = None
    size: Optional[Tuple[int, ...]] = None
    stride: Optional[Tuple[int, ...]] = None


class KJTList(Multistreamable):
    """One KJT per table group of a sharding."""

    def __init__(self, features: List[KeyedJaggedTensor]) -> None:
        self.features = features

    def __len__(self) -> int:
        return len(self.features)

    def __setitem__(self, key: int, item: KeyedJaggedTensor) -> None:
        self.features[key] = item

    def __getitem__(self, key: int) -> KeyedJaggedTensor:
        return self.features[key]

    def __iter__(self) -> Iterator[KeyedJaggedTensor]:
        return iter(self.features)

    def record_stream(self, stream: torch.Stream) -> None:
        for f in self.features:
            f.record_stream(stream)

    def __fx_create_arg__(self, tracer):
        return fx.node.Node  # pragma: no cover


@dataclass
class InputDistOutputs(Multistreamable):
    features: KJTList
    unbucketize_permute_tensor: Optional[torch.Tensor] = None
    bucket_mapping_tensor: Optional[torch.Tensor] = None
    bucketized_length: Optional[torch.Tensor] = None

    def record_stream(self, stream: torch.Stream) -> None:
        for t in (self.unbucketize_permute_tensor, self.bucket_mapping_tensor, self.bucketized_length):
            if t is not None and t.is_cuda:
                t.record_stream(stream)


class ListOfKJTList(Multistreamable):
    def __init__(self, features: List[KJTList]) -> None:
        self.features_list = features

    def __len__(self) -> int:
        return len(self.features_list)

    def __setitem__(self, key: int, item: KJTList) -> None:
        self.features_list[key] = item

    def __getitem__(self, key: int) -> KJTList:
        return self.features_list[key]

    def __iter__(self) -> Iterator[KJTList]:
        return iter(self.features_list)

    def record_stream(self, stream: torch.Stream) -> None:
        for f in self.features_list:
            f.record_stream(stream)


@dataclass
class ShardedConfig:
    local_rows: int = 0
    local_cols: int = 0


@dataclass
class ShardedMetaConfig(ShardedConfig):
    local_metadata: Optional[ShardMetadata] = None
    global_metadata: Optional[ShardedTensorMetadata] = None
    dtensor_metadata: Optional[Any] = None


@dataclass
class EmbeddingAttributes:
    compute_kernel: EmbeddingComputeKernel = EmbeddingComputeKernel.DENSE


@dataclass
class ShardedEmbeddingTable(ShardedMetaConfig, EmbeddingAttributes, EmbeddingTableConfig):
    """The piece of one table that lives on one rank."""

    fused_params: Optional[Dict[str, Any]] = None


@dataclass
class GroupedEmbeddingConfig:
    """Tables of one rank that share (dtype, pooling, weighted, kernel, optimizer) -> one TBE."""

    data_type: DataType
    pooling: PoolingType
    is_weighted: bool
    has_feature_processor: bool
    compute_kernel: EmbeddingComputeKernel
    embedding_tables: List[ShardedEmbeddingTable]
    fused_params: Optional[Dict[str, Any]] = None

    def feature_hash_sizes(self) -> List[int]:
        return [t.num_embeddings for t in self.embedding_tables for _ in range(t.num_features())]

    def feature_local_hash_sizes(self) -> List[int]:
        return [t.local_rows for t in self.embedding_tables for _ in range(t.num_features())]

    def num_features(self) -> int:
        return sum(t.num_features() for t in self.embedding_tables)

    def dim_sum(self) -> int:
        return sum(t.num_features() * t.local_cols for t in self.embedding_tables)

    def table_names(self) -> List[str]:
        return [t.name for t in self.embedding_tables]

    def feature_names(self) -> List[str]:
        return [f for t in self.embedding_tables for f in t.feature_names]

    def embedding_dims(self) -> List[int]:
        return [t.local_cols for t in self.embedding_tables for _ in t.feature_names]

    def embedding_names(self) -> List[str]:
        return [n for t in self.embedding_tables for n in t.embedding_names]

    def embedding_shard_metadata(self) -> List[Optional[ShardMetadata]]:
        return [t.local_metadata for t in self.embedding_tables for _ in t.feature_names]


F = TypeVar("F", bound=Multistreamable)
T = TypeVar("T")


class BaseEmbeddingLookup(abc.ABC, nn.Module, Generic[F, T]):
    @abc.abstractmethod
    def forward(self, sparse_features: F) -> T:
        ...


class FeatureShardingMixIn:
    def feature_names(self) -> List[str]:
        raise NotImplementedError

    def feature_names_per_rank(self) -> List[List[str]]:
        raise NotImplementedError

    def features_per_rank(self) -> List[int]:
        raise NotImplementedError


CompIn = TypeVar("CompIn")
DistOut = TypeVar("DistOut")
Out = TypeVar("Out")
ShrdCtx = TypeVar("ShrdCtx", bound=Multistreamable)


class ShardedEmbeddingModule(ShardedModule[CompIn, DistOut, Out, ShrdCtx]):
    """Base of the sharded embedding modules: owns lookups and exposes their fused optimizers."""

    def __init__(self, qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None) -> None:
        super().__init__(qcomm_codecs_registry)
        self._input_dists: List[nn.Module] = []
        self._lookups: List[nn.Module] = []
        self._output_dists: List[nn.Module] = []
        self.post_lookup_tracker_fn = None
        self.post_odist_tracker_fn = None

    def prefetch(self, dist_input, forward_stream=None, ctx=None) -> None:
        for feature, lookup in zip(dist_input, self._lookups):
            while isinstance(lookup, torch.nn.parallel.DistributedDataParallel):
                lookup = lookup.module
            if hasattr(lookup, "prefetch"):
                lookup.prefetch(sparse_features=feature, forward_stream=forward_stream)

    def extra_repr(self) -> str:
        def loop(key: str, modules: List[nn.Module]) -> List[str]:
            return [f"({key}): " + "\n".join(str(m) for m in modules)] if modules else []

        return "\n ".join(loop("lookups", self._lookups) + loop("_input_dists", self._input_dists) + loop("_output_dists", self._output_dists))

    def train(self, mode: bool = True):
        super().train(mode)
        for m in self._lookups:
            m.train(mode)
        return self

    @property
    def unsharded_module_type(self):
        raise NotImplementedError

    def register_post_lookup_tracker_fn(self, record_fn) -> None:
        self.post_lookup_tracker_fn = record_fn

    def register_post_odist_tracker_fn(self, record_fn) -> None:
        self.post_odist_tracker_fn = record_fn


M = TypeVar("M", bound=nn.Module)


class BaseEmbeddingSharder(ModuleSharder[M]):
    def __init__(self, fused_params: Optional[Dict[str, Any]] = None, qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None) -> None:
        super().__init__(qcomm_codecs_registry=qcomm_codecs_registry)
        self._fused_params = copy.deepcopy(fused_params) if fused_params is not None else fused_params
        self._fused_params_passed = fused_params is not None

    def sharding_types(self, compute_device_type: str) -> List[str]:
        types = [
            ShardingType.DATA_PARALLEL.value, ShardingType.TABLE_WISE.value, ShardingType.COLUMN_WISE.value,
            ShardingType.TABLE_COLUMN_WISE.value, ShardingType.ROW_WISE.value,
        ]
        if compute_device_type in {"cuda", "mtia"}:
            types += [ShardingType.TABLE_ROW_WISE.value, ShardingType.GRID_SHARD.value]
        return types

    def compute_kernels(self, sharding_type: str, compute_device_type: str) -> List[str]:
        ret: List[str] = []
        if sharding_type != ShardingType.DATA_PARALLEL.value:
            ret += [EmbeddingComputeKernel.FUSED.value]
            if compute_device_type in {"cuda"}:
                ret += [EmbeddingComputeKernel.FUSED_UVM.value, EmbeddingComputeKernel.FUSED_UVM_CACHING.value, EmbeddingComputeKernel.KEY_VALUE.value]
        else:
            ret.append(EmbeddingComputeKernel.DENSE.value)
        return ret

    @property
    def fused_params(self) -> Optional[Dict[str, Any]]:
        return self._fused_params

    def storage_usage(self, tensor: torch.Tensor, compute_device_type: str, compute_kernel: str) -> Dict[str, int]:
        tensor_bytes = get_tensor_size_bytes(tensor)
        if compute_kernel in {EmbeddingComputeKernel.FUSED_UVM.value, EmbeddingComputeKernel.FUSED_UVM_CACHING.value}:
            assert compute_device_type in {"cuda"}
            return {ParameterStorage.DDR.value: tensor_bytes}
        if compute_kernel in {EmbeddingComputeKernel.KEY_VALUE.value, EmbeddingComputeKernel.SSD_VIRTUAL_TABLE.value}:
            return {ParameterStorage.SSD.value: tensor_bytes}
        storage_map = {"cuda": ParameterStorage.HBM, "cpu": ParameterStorage.DDR, "mtia": ParameterStorage.DDR}
        return {storage_map[compute_device_type].value: tensor_bytes}


class BaseGroupedFeatureProcessor(nn.Module):
    @abc.abstractmethod
    def forward(self, features: KeyedJaggedTensor) -> KeyedJaggedTensor:
        ...


class BaseQuantEmbeddingSharder(ModuleSharder[M]):
    def __init__(self, fused_params: Optional[Dict[str, Any]] = None, shardable_params: Optional[List[str]] = None) -> None:
        super().__init__()
        self._fused_params = copy.deepcopy(fused_params) if fused_params is not None else fused_params
        self._shardable_params: List[str] = shardable_params if shardable_params else []

    def sharding_types(self, compute_device_type: str) -> List[str]:
        return [ShardingType.TABLE_WISE.value, ShardingType.ROW_WISE.value, ShardingType.COLUMN_WISE.value]

    def shardable_parameters(self, module: M) -> Dict[str, nn.Parameter]:
        shardable = {}
        for name, p in module.state_dict().items():
            if name.endswith(".weight"):
                tname = name.split(".")[-2]
                if not self._shardable_params or tname in self._shardable_params:
                    shardable[tname] = p
        return shardable

    def compute_kernels(self, sharding_type: str, compute_device_type: str) -> List[str]:
        ret = [EmbeddingComputeKernel.QUANT.value]
        if compute_device_type in {"cuda"}:
            ret += [EmbeddingComputeKernel.QUANT_UVM.value, EmbeddingComputeKernel.QUANT_UVM_CACHING.value]
        return ret

    @property
    def fused_params(self) -> Optional[Dict[str, Any]]:
        return self._fused_params

    def storage_usage(self, tensor: torch.Tensor, compute_device_type: str, compute_kernel: str) -> Dict[str, int]:
        tensor_bytes = get_tensor_size_bytes(tensor) + tensor.shape[0] * 4
        if compute_kernel in {EmbeddingComputeKernel.QUANT_UVM.value, EmbeddingComputeKernel.QUANT_UVM_CACHING.value}:
            return {ParameterStorage.DDR.value: tensor_bytes}
        storage_map = {"cuda": ParameterStorage.HBM, "cpu": ParameterStorage.DDR, "mtia": ParameterStorage.DDR}
        return {storage_map[compute_device_type].value: tensor_bytes}
