"""Embedding-table schemas and the enums that describe them.

API counterpart of ``torchrec/modules/embedding_configs.py:26-436`` in the reference.
The kernel-side enums (``PoolingMode``, ``SparseType``) that the reference imports from
an external wheel are defined here because the kernels live in this repository.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum, IntEnum, unique
from functools import partial
from math import sqrt
from typing import Callable, Dict, List, NamedTuple, Optional

import torch

from torchrec_b200.types import DataType


@unique
class PoolingType(Enum):
    SUM = "SUM"
    MEAN = "MEAN"
    NONE = "NONE"


class PoolingMode(IntEnum):
    """Pooling performed by the table-batched embedding kernels."""

    SUM = 0
    MEAN = 1
    NONE = 2


class SparseType(Enum):
    FP32 = "fp32"
    FP16 = "fp16"
    BF16 = "bf16"
    FP8 = "fp8"
    INT8 = "int8"
    INT4 = "int4"
    INT2 = "int2"
    NFP8 = "nfp8"

    def bit_rate(self) -> int:
        return {"fp32": 32, "fp16": 16, "bf16": 16, "fp8": 8, "int8": 8, "int4": 4, "int2": 2, "nfp8": 8}[self.value]

    def as_dtype(self) -> torch.dtype:
        return {
            "fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16, "fp8": torch.uint8,
            "int8": torch.uint8, "int4": torch.quint4x2, "int2": torch.quint2x4, "nfp8": torch.float8_e4m3fn,
        }[self.value]


class _ShardingTypeForPooling(Enum):
    ROW_WISE = "row_wise"
    TABLE_ROW_WISE = "table_row_wise"
    GRID_SHARD = "grid_shard"


DATA_TYPE_NUM_BITS: Dict[DataType, int] = {
    DataType.FP32: 32,
    DataType.FP16: 16,
    DataType.BF16: 16,
    DataType.INT8: 8,
    DataType.UINT8: 8,
    DataType.INT4: 4,
    DataType.INT2: 2,
    DataType.NFP8: 8,
}


def dtype_to_data_type(dtype: torch.dtype) -> DataType:
    table = {
        torch.float: DataType.FP32, torch.float32: DataType.FP32,
        torch.float16: DataType.FP16, torch.half: DataType.FP16, torch.bfloat16: DataType.BF16,
        torch.int8: DataType.INT8, torch.qint8: DataType.INT8, torch.uint8: DataType.UINT8, torch.quint8: DataType.UINT8,
        torch.quint4x2: DataType.INT4, torch.quint2x4: DataType.INT2, torch.float8_e4m3fn: DataType.NFP8,
        torch.int64: DataType.INT64, torch.long: DataType.INT64, torch.int32: DataType.INT32, torch.int: DataType.INT32,
    }
    if dtype not in table:
        raise Exception(f"Invalid data type {dtype}")
    return table[dtype]


def pooling_type_to_pooling_mode(pooling_type: PoolingType, sharding_type=None) -> PoolingMode:
    """MEAN becomes SUM for row-split shardings: the divisor needs the bag length over all
    shards, so it is applied after the reduction (``torchrec/modules/embedding_configs.py:98-113``)."""
    if pooling_type.value == PoolingType.SUM.value:
        return PoolingMode.SUM
    if pooling_type.value == PoolingType.MEAN.value:
        if sharding_type is not None and getattr(sharding_type, "value", sharding_type) in ("row_wise", "table_row_wise", "grid_shard"):
            return PoolingMode.SUM
        return PoolingMode.MEAN
    if pooling_type.value == PoolingType.NONE.value:
        return PoolingMode.NONE
    raise Exception(f"Invalid pooling type {pooling_type}")


def pooling_type_to_str(pooling_type: PoolingType) -> str:
    if pooling_type.value == PoolingType.SUM.value:
        return "sum"
    if pooling_type.value == PoolingType.MEAN.value:
        return "mean"
    raise ValueError(f"Unsupported pooling type {pooling_type}")


def data_type_to_sparse_type(data_type: DataType) -> SparseType:
    m = {
        DataType.FP32: SparseType.FP32, DataType.FP16: SparseType.FP16, DataType.BF16: SparseType.BF16,
        DataType.INT8: SparseType.INT8, DataType.UINT8: SparseType.INT8, DataType.INT4: SparseType.INT4,
        DataType.INT2: SparseType.INT2, DataType.NFP8: SparseType.NFP8,
    }
    if data_type not in m:
        raise ValueError(f"Invalid DataType {data_type}")
    return m[data_type]


def data_type_to_dtype(data_type: DataType) -> torch.dtype:
    m = {
        "FP32": torch.float32, "FP16": torch.float16, "BF16": torch.bfloat16, "NFP8": torch.float8_e4m3fn,
        "INT64": torch.int64, "INT32": torch.int32, "INT8": torch.int8, "UINT8": torch.uint8,
        "INT4": torch.quint4x2, "INT2": torch.quint2x4,
    }
    if data_type.value not in m:
        raise ValueError(f"DataType {data_type} cannot be converted to dtype")
    return m[data_type.value]


# ---- virtual-table eviction policies (configuration only) ----------------------------
@dataclass
class VirtualTableEvictionPolicy:
    """Base of the eviction policies attached to virtual (unbounded-id) tables."""

    inference_eviction_threshold: Optional[float] = None
    initialized: bool = False

    def init_metaheader_config(self, data_type: DataType, embedding_dim: int) -> None:
        self.initialized = True

    def get_meta_header_len(self) -> int:
        return 0


@dataclass
class NoEvictionPolicy(VirtualTableEvictionPolicy):
    pass


@dataclass
class CountBasedEvictionPolicy(VirtualTableEvictionPolicy):
    training_id_eviction_trigger_count: Optional[int] = None
    training_id_keep_count: Optional[int] = None
    eviction_threshold: int = 0
    decay_rate: float = 0.99


@dataclass
class TimestampBasedEvictionPolicy(VirtualTableEvictionPolicy):
    training_id_eviction_trigger_count: Optional[int] = None
    training_id_keep_count: Optional[int] = None
    eviction_ttl_mins: int = 0


@dataclass
class CountTimestampMixedEvictionPolicy(VirtualTableEvictionPolicy):
    training_id_eviction_trigger_count: Optional[int] = None
    training_id_keep_count: Optional[int] = None
    eviction_threshold: int = 0
    decay_rate: float = 0.99
    eviction_ttl_mins: int = 0


@dataclass
class FeatureL2NormBasedEvictionPolicy(VirtualTableEvictionPolicy):
    training_id_eviction_trigger_count: Optional[int] = None
    training_id_keep_count: Optional[int] = None
    eviction_threshold: float = 0.0


@dataclass
class FeatureScoreBasedEvictionPolicy(VirtualTableEvictionPolicy):
    training_id_eviction_trigger_count: Optional[int] = None
    training_id_keep_count: Optional[int] = None
    target_eviction_percent: float = 0.0
    eviction_ttl_mins: int = 0


@dataclass
class BaseEmbeddingConfig:
    """Schema of one embedding table.

    Default initialisation is ``U(-sqrt(1/num_embeddings), +sqrt(1/num_embeddings))``.
    """

    num_embeddings: int
    embedding_dim: int
    name: str = ""
    data_type: DataType = DataType.FP32
    feature_names: List[str] = field(default_factory=list)
    weight_init_max: Optional[float] = None
    weight_init_min: Optional[float] = None
    num_embeddings_post_pruning: Optional[int] = None
    init_fn: Optional[Callable[[torch.Tensor], Optional[torch.Tensor]]] = None
    need_pos: bool = False
    input_dim: Optional[int] = None
    total_num_buckets: Optional[int] = None
    use_virtual_table: bool = False
    virtual_table_eviction_policy: Optional[VirtualTableEvictionPolicy] = None
    enable_embedding_update: bool = False

    def get_weight_init_max(self) -> float:
        return sqrt(1 / self.num_embeddings) if self.weight_init_max is None else self.weight_init_max

    def get_weight_init_min(self) -> float:
        return -sqrt(1 / self.num_embeddings) if self.weight_init_min is None else self.weight_init_min

    def num_features(self) -> int:
        return len(self.feature_names)

    def __post_init__(self) -> None:
        if self.init_fn is None:
            self.init_fn = partial(torch.nn.init.uniform_, a=self.get_weight_init_min(), b=self.get_weight_init_max())


@dataclass
class EmbeddingTableConfig(BaseEmbeddingConfig):
    pooling: PoolingType = PoolingType.SUM
    is_weighted: bool = False
    has_feature_processor: bool = False
    embedding_names: List[str] = field(default_factory=list)


@dataclass
class EmbeddingBagConfig(BaseEmbeddingConfig):
    """A table whose lookups are pooled per bag."""

    pooling: PoolingType = PoolingType.SUM


@dataclass
class EmbeddingConfig(BaseEmbeddingConfig):
    """A table whose lookups are returned per id (sequence embeddings)."""

    pass


class QuantConfig(NamedTuple):
    activation: object
    weight: object
    per_table_weight_dtype: Optional[Dict[str, torch.dtype]] = None
