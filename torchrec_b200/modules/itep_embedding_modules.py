"""Embedding collections whose ids pass through an in-training-pruning module first.
Counterpart of ``torchrec/modules/itep_embedding_modules.py`` (``ITEPEmbeddingBagCollection`` ``:27``, ``ITEPEmbeddingCollection``)."""
from __future__ import annotations

from typing import Dict

import torch
from torch import nn

from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection, EmbeddingCollection
from torchrec_b200.modules.itep_modules import GenericITEPModule
from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor, KeyedTensor


class ITEPEmbeddingBagCollection(nn.Module):
    def __init__(self, embedding_bag_collection: EmbeddingBagCollection, itep_module: GenericITEPModule) -> None:
        super().__init__()
        self._embedding_bag_collection = embedding_bag_collection
        self._itep_module = itep_module
        # on the host: it steers the schedule and is checkpointed
        self.register_buffer("_iter", torch.tensor(0, dtype=torch.int64, device=torch.device("cpu")))

    def forward(self, features: KeyedJaggedTensor) -> KeyedTensor:
        features = self._itep_module(features, int(self._iter.item()))
        pooled = self._embedding_bag_collection(features)
        self._iter += 1
        return pooled


class ITEPEmbeddingCollection(nn.Module):
    def __init__(self, embedding_collection: EmbeddingCollection, itep_module: GenericITEPModule) -> None:
        super().__init__()
        self._embedding_collection = embedding_collection
        self._itep_module = itep_module
        self.register_buffer("_iter", torch.tensor(0, dtype=torch.int64, device=torch.device("cpu")))

    def forward(self, features: KeyedJaggedTensor) -> Dict[str, JaggedTensor]:
        features = self._itep_module(features, int(self._iter.item()))
        out = self._embedding_collection(features)
        self._iter += 1
        return out
