"""Metadata records written into a module's ``ir_metadata`` buffer as JSON (``torchrec/ir/schema.py``)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

from torchrec_b200.modules.embedding_configs import DataType, PoolingType


@dataclass
class EmbeddingBagConfigMetadata:
    num_embeddings: int
    embedding_dim: int
    name: str
    data_type: DataType
    feature_names: List[str]
    weight_init_max: Optional[float]
    weight_init_min: Optional[float]
    need_pos: bool
    pooling: PoolingType


@dataclass
class EBCMetadata:
    tables: List[EmbeddingBagConfigMetadata]
    is_weighted: bool
    device: Optional[str]


@dataclass
class FPEBCMetadata:
    is_fp_collection: bool
    features: List[str]


@dataclass
class PositionWeightedModuleMetadata:
    max_feature_length: int


@dataclass
class PositionWeightedModuleCollectionMetadata:
    max_feature_lengths: List[Tuple[str, int]]


@dataclass
class KTRegroupAsDictMetadata:
    groups: List[List[str]]
    keys: List[str]
    emb_dtype: Optional[str]
