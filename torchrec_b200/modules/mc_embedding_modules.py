"""Embedding collections behind a managed-collision remapper: ids are remapped, rows whose slot changed owner are reset
to the table's initial distribution, then looked up (``torchrec/modules/mc_embedding_modules.py``)."""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple, Union

import torch
from torch import nn

from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection, EmbeddingCollection
from torchrec_b200.modules.mc_modules import ManagedCollisionCollection
from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor, KeyedTensor


def evict(evictions: Dict[str, Optional[torch.Tensor]], ebc: Union[EmbeddingBagCollection, EmbeddingCollection]) -> None:
    """Re-initialise the rows listed per table."""
    container = ebc.embedding_bags if isinstance(ebc, EmbeddingBagCollection) else ebc.embeddings
    configs = ebc.embedding_bag_configs() if isinstance(ebc, EmbeddingBagCollection) else ebc.embedding_configs()
    by_name = {c.name: c for c in configs}
    for table, rows in evictions.items():
        if rows is None or rows.numel() == 0:
            continue
        w = container[table].weight
        cfg = by_name[table]
        lo, hi = cfg.get_weight_init_min(), cfg.get_weight_init_max()
        with torch.no_grad():
            w[rows.to(w.device)] = torch.empty(rows.numel(), w.shape[1], device=w.device, dtype=w.dtype).uniform_(lo, hi)


class BaseManagedCollisionEmbeddingCollection(nn.Module):
    def __init__(self, embedding_module: Union[EmbeddingBagCollection, EmbeddingCollection], managed_collision_collection: ManagedCollisionCollection,
                 return_remapped_features: bool = False) -> None:
        super().__init__()
        self._managed_collision_collection = managed_collision_collection
        self._return_remapped_features = return_remapped_features
        self._embedding_module = embedding_module

    def forward(self, features: KeyedJaggedTensor) -> Tuple[Union[KeyedTensor, Dict[str, JaggedTensor]], Optional[KeyedJaggedTensor]]:
        remapped = self._managed_collision_collection(features)
        evict(self._managed_collision_collection.evict(), self._embedding_module)
        out = self._embedding_module(remapped)
        return out, (remapped if self._return_remapped_features else None)


class ManagedCollisionEmbeddingCollection(BaseManagedCollisionEmbeddingCollection):
    def __init__(self, embedding_collection: EmbeddingCollection, managed_collision_collection: ManagedCollisionCollection, return_remapped_features: bool = False) -> None:
        super().__init__(embedding_collection, managed_collision_collection, return_remapped_features)


class ManagedCollisionEmbeddingBagCollection(BaseManagedCollisionEmbeddingCollection):
    def __init__(self, embedding_bag_collection: EmbeddingBagCollection, managed_collision_collection: ManagedCollisionCollection, return_remapped_features: bool = False) -> None:
        super().__init__(embedding_bag_collection, managed_collision_collection, return_remapped_features)
