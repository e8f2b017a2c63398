"""Unsharded embedding collections -- the single-device semantics every sharded path must match.

Counterpart of ``torchrec/modules/embedding_modules.py:97-543``.  ``EmbeddingBagCollection``
pools ids per bag and returns a ``KeyedTensor``; ``EmbeddingCollection`` returns the
per-id rows as a dict of ``JaggedTensor``.  Parameter names
(``embedding_bags.<table>.weight`` / ``embeddings.<table>.weight``) are the checkpoint keys
and do not change when the module is sharded.
"""
from __future__ import annotations

import abc
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from torchrec_b200.modules.embedding_configs import (
    DataType,
    EmbeddingBagConfig,
    EmbeddingConfig,
    data_type_to_dtype,
    pooling_type_to_str,
)
from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor, KeyedTensor


def reorder_inverse_indices(inverse_indices: Optional[Tuple[List[str], torch.Tensor]], feature_names: List[str]) -> torch.Tensor:
    if inverse_indices is None:
        return torch.empty(0)
    index_per_name = {name: i for i, name in enumerate(inverse_indices[0])}
    index = torch.tensor([index_per_name[n] for n in feature_names if n in index_per_name], device=inverse_indices[1].device)
    return torch.index_select(inverse_indices[1], 0, index)


def process_pooled_embeddings(pooled_embeddings: List[torch.Tensor], inverse_indices: torch.Tensor) -> torch.Tensor:
    """Concatenate per-feature pooled outputs; with variable batch per feature each output is
    first expanded back to the full batch through its row of ``inverse_indices``."""
    if inverse_indices.numel() > 0:
        pooled_embeddings = [
            emb.index_select(0, inverse_indices[i].to(torch.int64)) for i, emb in enumerate(pooled_embeddings)
        ]
    return torch.cat(pooled_embeddings, dim=1)


def get_embedding_names_by_table(tables) -> List[List[str]]:
    """A feature used by more than one table is exposed as ``feature@table``."""
    shared_feature: Dict[str, bool] = {}
    for cfg in tables:
        for f in cfg.feature_names:
            shared_feature[f] = f in shared_feature
    out: List[List[str]] = []
    for cfg in tables:
        out.append([f + "@" + cfg.name if shared_feature[f] else f for f in cfg.feature_names])
    return out


def _reject_duplicate_names(tables) -> None:
    seen = set()
    for cfg in tables:
        if cfg.name in seen:
            raise ValueError(f"Duplicate table name {cfg.name}")
        seen.add(cfg.name)


def _table_dtype(cfg) -> torch.dtype:
    return torch.float32 if cfg.data_type == DataType.FP32 else data_type_to_dtype(cfg.data_type)


class EmbeddingBagCollectionInterface(abc.ABC, nn.Module):
    @abc.abstractmethod
    def forward(self, features: KeyedJaggedTensor) -> KeyedTensor:
        ...

    @abc.abstractmethod
    def embedding_bag_configs(self) -> List[EmbeddingBagConfig]:
        ...

    @abc.abstractmethod
    def is_weighted(self) -> bool:
        ...


class EmbeddingBagCollection(EmbeddingBagCollectionInterface):
    """A set of pooled embedding tables addressed by feature name.

    ``forward(KeyedJaggedTensor) -> KeyedTensor`` with ``values [B, sum(D over features)]``
    in table order (features of table 0 first).
    """

    def __init__(
        self,
        tables: List[EmbeddingBagConfig],
        is_weighted: bool = False,
        device: Optional[torch.device] = None,
    ) -> None:
        super().__init__()
        _reject_duplicate_names(tables)
        self._is_weighted, self._embedding_bag_configs = is_weighted, tables
        for cfg in tables:
            cfg.feature_names = cfg.feature_names or [cfg.name]
        self.embedding_bags = nn.ModuleDict({
            cfg.name: nn.EmbeddingBag(cfg.num_embeddings, cfg.embedding_dim, mode=pooling_type_to_str(cfg.pooling), device=device,
                                      include_last_offset=True, dtype=_table_dtype(cfg))
            for cfg in tables
        })
        if device is None and tables:
            device = self.embedding_bags[tables[0].name].weight.device
        self._device: torch.device = torch.device("cpu") if device is None else device
        self._lengths_per_embedding: List[int] = [cfg.embedding_dim for cfg in tables for _ in cfg.feature_names]
        self._embedding_names: List[str] = [n for names in get_embedding_names_by_table(tables) for n in names]
        self._feature_names: List[List[str]] = [cfg.feature_names for cfg in tables]
        self.reset_parameters()

    def forward(self, features: KeyedJaggedTensor) -> KeyedTensor:
        inverse_indices = reorder_inverse_indices(features.inverse_indices_or_none(), [f for names in self._feature_names for f in names])
        per_feature = features.to_dict()
        pooled: List[torch.Tensor] = []
        for bag, features_of_table in zip(self.embedding_bags.values(), self._feature_names):
            for feature in features_of_table:
                jt = per_feature[feature]
                weights = jt.weights().to(bag.weight.dtype) if self._is_weighted else None
                pooled.append(bag(jt.values(), jt.offsets(), per_sample_weights=weights).float())
        return KeyedTensor(keys=self._embedding_names, values=process_pooled_embeddings(pooled, inverse_indices),
                           length_per_key=self._lengths_per_embedding)

    def is_weighted(self) -> bool:
        return self._is_weighted

    def embedding_bag_configs(self) -> List[EmbeddingBagConfig]:
        return self._embedding_bag_configs

    @property
    def device(self) -> torch.device:
        return self._device

    def reset_parameters(self) -> None:
        if (isinstance(self.device, torch.device) and self.device.type == "meta") or (
            isinstance(self.device, str) and self.device == "meta"
        ):
            return
        for cfg in self._embedding_bag_configs:
            assert cfg.init_fn is not None
            param = self.embedding_bags[cfg.name].weight
            cfg.init_fn(param)


class EmbeddingCollectionInterface(abc.ABC, nn.Module):
    @abc.abstractmethod
    def forward(self, features: KeyedJaggedTensor) -> Dict[str, JaggedTensor]:
        ...

    @abc.abstractmethod
    def embedding_configs(self) -> List[EmbeddingConfig]:
        ...

    @abc.abstractmethod
    def need_indices(self) -> bool:
        ...

    @abc.abstractmethod
    def embedding_dim(self) -> int:
        ...

    @abc.abstractmethod
    def embedding_names_by_table(self) -> List[List[str]]:
        ...


class EmbeddingCollection(EmbeddingCollectionInterface):
    """A set of unpooled (sequence) embedding tables; every table has the same dim.

    ``forward(KeyedJaggedTensor) -> Dict[feature, JaggedTensor]`` where each JT holds the
    looked-up rows ``[sum L, D]`` with the input lengths.
    """

    def __init__(
        self,
        tables: List[EmbeddingConfig],
        device: Optional[torch.device] = None,
        need_indices: bool = False,
    ) -> None:
        super().__init__()
        self._embedding_configs = tables
        self._need_indices: bool = need_indices
        self._device: torch.device = torch.device("cpu") if device is None else device
        names = [t.name for t in tables]
        repeated = [n for n in names if names.count(n) > 1]
        if repeated:
            raise ValueError(f"Duplicate table name {repeated[0]}")
        dims = {t.embedding_dim for t in tables}
        self._embedding_dim: int = tables[0].embedding_dim if tables else -1
        if len(dims) > 1:
            odd = next(t for t in tables if t.embedding_dim != self._embedding_dim)
            raise ValueError(
                "All tables in a EmbeddingCollection are required to have same embedding dimension."
                + f" Violating case: {odd.name}'s embedding_dim {odd.embedding_dim} != {self._embedding_dim}"
            )
        self.embeddings: nn.ModuleDict = nn.ModuleDict()
        for t in tables:
            t.feature_names = t.feature_names or [t.name]
            self.embeddings[t.name] = nn.Embedding(t.num_embeddings, t.embedding_dim, device=device,
                                                   dtype=torch.float32 if t.data_type == DataType.FP32 else data_type_to_dtype(t.data_type))
        self._embedding_names_by_table: List[List[str]] = get_embedding_names_by_table(tables)
        self._feature_names: List[List[str]] = [t.feature_names for t in tables]
        self.reset_parameters()

    def forward(self, features: KeyedJaggedTensor) -> Dict[str, JaggedTensor]:
        per_feature = features.to_dict()
        out: Dict[str, JaggedTensor] = {}
        for table, feats, emb_names in zip(self.embeddings.values(), self._feature_names, self._embedding_names_by_table):
            for feat, emb_name in zip(feats, emb_names):
                jt = per_feature[feat]
                ids = jt.values()
                out[emb_name] = JaggedTensor(values=table(ids).float(), lengths=jt.lengths(), weights=ids if self._need_indices else None)
        return out

    def need_indices(self) -> bool:
        ...

    @abc.abstractmethod
    def embedding_dim(self) -> int:
        ...

    @abc.abstractmethod
    def embedding_names_by_table(self) -> List[List[str]]:
        ...


class EmbeddingCollection(EmbeddingCollectionInterface):
    """A set of unpooled (sequence) embedding tables; every table has the same dim.

    ``forward(KeyedJaggedTensor) -> Dict[feature, JaggedTensor]`` where each JT holds the
    looked-up rows ``[sum L, D]`` with the input lengths.
    """

    def __init__(
        self,
        tables: List[EmbeddingConfig],
        device: Optional[torch.device] = None,
        need_indices: bool = False,
    ) -> None:
        super().__init__()
        _reject_duplicate_names(tables)
        dims = {cfg.embedding_dim for cfg in tables}
        if len(dims) > 1:
            first = tables[0].embedding_dim
            odd = next(cfg for cfg in tables if cfg.embedding_dim != first)
            raise ValueError("All tables in a EmbeddingCollection are required to have same embedding dimension."
                             f" Violating case: {odd.name}'s embedding_dim {odd.embedding_dim} != {first}")
        self._embedding_configs, self._need_indices = tables, need_indices
        self._embedding_dim: int = dims.pop() if dims else -1
        self._device: torch.device = torch.device("cpu") if device is None else device
        self.embeddings = nn.ModuleDict({
            cfg.name: nn.Embedding(cfg.num_embeddings, cfg.embedding_dim, device=device, dtype=_table_dtype(cfg)) for cfg in tables
        })
        for cfg in tables:
            cfg.feature_names = cfg.feature_names or [cfg.name]
        self._embedding_names_by_table: List[List[str]] = get_embedding_names_by_table(tables)
        self._feature_names: List[List[str]] = [cfg.feature_names for cfg in tables]
        self.reset_parameters()

    def forward(self, features: KeyedJaggedTensor) -> Dict[str, JaggedTensor]:
        per_feature = features.to_dict()
        out: Dict[str, JaggedTensor] = {}
        for table, features_of_table, names_of_table in zip(self.embeddings.values(), self._feature_names, self._embedding_names_by_table):
            for feature, name in zip(features_of_table, names_of_table):
                jt = per_feature[feature]
                ids = jt.values()
                out[name] = JaggedTensor(values=table(ids).float(), lengths=jt.lengths(), weights=ids if self._need_indices else None)
        return out

    def need_indices(self) -> bool:
        return self._need_indices

    def embedding_dim(self) -> int:
        return self._embedding_dim

    def embedding_configs(self) -> List[EmbeddingConfig]:
        return self._embedding_configs

    def embedding_names_by_table(self) -> List[List[str]]:
        return self._embedding_names_by_table

    @property
    def device(self) -> torch.device:
        return self._device

    def reset_parameters(self) -> None:
        if isinstance(self.device, torch.device) and self.device.type == "meta":
            return
        for cfg in self._embedding_configs:
            assert cfg.init_fn is not None
            cfg.init_fn(self.embeddings[cfg.name].weight)
