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
        self._is_weighted = is_weighted
        self.embedding_bags: nn.ModuleDict = nn.ModuleDict()
        self._embedding_bag_configs = tables
        self._lengths_per_embedding: List[int] = []
        self._dtypes: List[int] = []
        table_names = set()
        for cfg in tables:
            if cfg.name in table_names:
                raise ValueError(f"Duplicate table name {cfg.name}")
            table_names.add(cfg.name)
            dtype = torch.float32 if cfg.data_type == DataType.FP32 else data_type_to_dtype(cfg.data_type)
            self.embedding_bags[cfg.name] = nn.EmbeddingBag(
                num_embeddings=cfg.num_embeddings,
                embedding_dim=cfg.embedding_dim,
                mode=pooling_type_to_str(cfg.pooling),
                device=device,
                include_last_offset=True,
                dtype=dtype,
            )
            if device is None:
                device = self.embedding_bags[cfg.name].weight.device
            if not cfg.feature_names:
                cfg.feature_names = [cfg.name]
            self._lengths_per_embedding.extend(len(cfg.feature_names) * [cfg.embedding_dim])
        self._device: torch.device = device if device is not None else torch.device("cpu")
        self._embedding_names: List[str] = [n for names in get_embedding_names_by_table(tables) for n in names]
        self._feature_names: List[List[str]] = [t.feature_names for t in tables]
        self.reset_parameters()

    def forward(self, features: KeyedJaggedTensor) -> KeyedTensor:
        flat_feature_names = [n for names in self._feature_names for n in names]
        inverse_indices = reorder_inverse_indices(features.inverse_indices_or_none(), flat_feature_names)
        pooled: List[torch.Tensor] = []
        feature_dict = features.to_dict()
        for i, bag in enumerate(self.embedding_bags.values()):
            for feature_name in self._feature_names[i]:
                f = feature_dict[feature_name]
                w = f.weights() if self._is_weighted else None
                if w is not None and w.dtype != bag.weight.dtype:
                    w = w.to(bag.weight.dtype)
                res = bag(input=f.values(), offsets=f.offsets(), per_sample_weights=w).float()
                pooled.append(res)
        return KeyedTensor(
            keys=self._embedding_names,
            values=process_pooled_embeddings(pooled, inverse_indices),
            length_per_key=self._lengths_per_embedding,
        )

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
        self.embeddings: nn.ModuleDict = nn.ModuleDict()
        self._embedding_configs = tables
        self._embedding_dim: int = -1
        self._need_indices: bool = need_indices
        self._device: torch.device = device if device is not None else torch.device("cpu")
        table_names = set()
        for config in tables:
            if config.name in table_names:
                raise ValueError(f"Duplicate table name {config.name}")
            table_names.add(config.name)
            self._embedding_dim = config.embedding_dim if self._embedding_dim < 0 else self._embedding_dim
            if self._embedding_dim != config.embedding_dim:
                raise ValueError(
                    "All tables in a EmbeddingCollection are required to have same embedding dimension."
                    + f" Violating case: {config.name}'s embedding_dim {config.embedding_dim} != {self._embedding_dim}"
                )
            dtype = torch.float32 if config.data_type == DataType.FP32 else data_type_to_dtype(config.data_type)
            self.embeddings[config.name] = nn.Embedding(
                num_embeddings=config.num_embeddings, embedding_dim=config.embedding_dim, device=device, dtype=dtype,
            )
            if not config.feature_names:
                config.feature_names = [config.name]
        self._embedding_names_by_table: List[List[str]] = get_embedding_names_by_table(tables)
        self._feature_names: List[List[str]] = [t.feature_names for t in tables]
        self.reset_parameters()

    def forward(self, features: KeyedJaggedTensor) -> Dict[str, JaggedTensor]:
        feature_embeddings: Dict[str, JaggedTensor] = {}
        jt_dict = features.to_dict()
        for i, emb_module in enumerate(self.embeddings.values()):
            feature_names = self._feature_names[i]
            embedding_names = self._embedding_names_by_table[i]
            for j, embedding_name in enumerate(embedding_names):
                f = jt_dict[feature_names[j]]
                lookup = emb_module(input=f.values()).float()
                feature_embeddings[embedding_name] = JaggedTensor(
                    values=lookup, lengths=f.lengths(), weights=f.values() if self._need_indices else None,
                )
        return feature_embeddings

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
