"""Metadata records that travel in a module's ``ir_metadata`` buffer as JSON.

Each record type is declared as a table of ``field -> type`` and turned into a dataclass, so the JSON keys, their order and the
constructor signature come from one place.  Enum-valued fields (``data_type``, ``pooling``) are stored by value.  The key set equals
the reference's ``torchrec/ir/schema.py`` so that metadata written by either framework can be read by the other.
"""
from __future__ import annotations

from dataclasses import make_dataclass
from typing import Any, Dict, List, Optional, Tuple

from torchrec_b200.modules.embedding_configs import DataType, PoolingType


def _record(name: str, fields: Dict[str, Any], doc: str) -> type:
    cls = make_dataclass(name, list(fields.items()))
    cls.__doc__ = doc
    cls.__module__ = __name__
    return cls


EmbeddingBagConfigMetadata = _record(
    "EmbeddingBagConfigMetadata",
    {"num_embeddings": int, "embedding_dim": int, "name": str, "data_type": DataType, "feature_names": List[str], "weight_init_max": Optional[float],
     "weight_init_min": Optional[float], "need_pos": bool, "pooling": PoolingType},
    "One embedding-bag table.")

EBCMetadata = _record(
    "EBCMetadata", {"tables": List[EmbeddingBagConfigMetadata], "is_weighted": bool, "device": Optional[str]},
    "An ``EmbeddingBagCollection``: its tables, whether lookups are weighted, and the device it was built on.")

FPEBCMetadata = _record(
    "FPEBCMetadata", {"is_fp_collection": bool, "features": List[str]},
    "A feature-processed collection: one processor collection, or one processor per listed feature.")

PositionWeightedModuleMetadata = _record("PositionWeightedModuleMetadata", {"max_feature_length": int}, "Position weights of one feature.")

PositionWeightedModuleCollectionMetadata = _record(
    "PositionWeightedModuleCollectionMetadata", {"max_feature_lengths": List[Tuple[str, int]]}, "Position weights of several features, as (feature, length) pairs.")

KTRegroupAsDictMetadata = _record(
    "KTRegroupAsDictMetadata", {"groups": List[List[str]], "keys": List[str], "emb_dtype": Optional[str]}, "A keyed-tensor regroup: the groups, their output keys, an optional cast.")
