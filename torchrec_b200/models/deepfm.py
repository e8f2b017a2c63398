"""DeepFM recommendation model: pooled sparse embeddings and a projected dense vector feed a deep branch (one linear + ReLU over
the flattened concatenation) and a second-order factorization-machine term; the over arch is a linear layer with a sigmoid.
Counterpart of ``torchrec/models/deepfm.py:20-385``."""
from __future__ import annotations

from typing import List, Optional, Tuple, Union

import torch
from torch import nn

from torchrec_b200.modules.deepfm import DeepFM, FactorizationMachine
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor, KeyedTensor


class SparseArch(nn.Module):
    """Pooled lookup of every sparse feature: KJT -> KeyedTensor ``[B, sum(D)]``."""

    def __init__(self, embedding_bag_collection: EmbeddingBagCollection) -> None:
        super().__init__()
        self.embedding_bag_collection: EmbeddingBagCollection = embedding_bag_collection

    def forward(self, features: KeyedJaggedTensor) -> KeyedTensor:
        return self.embedding_bag_collection(features)


class DenseArch(nn.Module):
    """Two linear + ReLU layers: ``[B, in_features]`` -> ``[B, embedding_dim]``."""

    def __init__(self, in_features: int, hidden_layer_size: int, embedding_dim: int) -> None:
        super().__init__()
        self.model: nn.Module = nn.Sequential(nn.Linear(in_features, hidden_layer_size), nn.ReLU(), nn.Linear(hidden_layer_size, embedding_dim), nn.ReLU())

    def forward(self, features: torch.Tensor) -> torch.Tensor:
        return self.model(features)


class FMInteractionArch(nn.Module):
    """``[dense, deep(dense ++ sparse), fm(dense ++ sparse)]`` -> ``[B, D + deep_fm_dimension + 1]``; with no sparse feature the
    dense vector passes through."""

    def __init__(self, fm_in_features: int, sparse_feature_names: List[str], deep_fm_dimension: int) -> None:
        super().__init__()
        self.sparse_feature_names: List[str] = sparse_feature_names
        self.deep_fm = DeepFM(dense_module=nn.Sequential(nn.Linear(fm_in_features, deep_fm_dimension), nn.ReLU()))
        self.fm = FactorizationMachine()

    def forward(self, dense_features: torch.Tensor, sparse_features: KeyedTensor) -> torch.Tensor:
        if not self.sparse_feature_names:
            return dense_features
        per_key = sparse_features.to_dict()
        parts = [dense_features] + [per_key[name] for name in self.sparse_feature_names]
        return torch.cat([dense_features, self.deep_fm(parts), self.fm(parts)], dim=1)


class OverArch(nn.Module):
    """Linear to one unit followed by a sigmoid: the output is a probability, not a logit."""

    def __init__(self, in_features: int) -> None:
        super().__init__()
        self.model: nn.Module = nn.Sequential(nn.Linear(in_features, 1), nn.Sigmoid())

    def forward(self, features: torch.Tensor) -> torch.Tensor:
        return self.model(features)


class SimpleDeepFMNN(nn.Module):
    """Dense arch + sparse arch + FM interaction + over arch.  Every table must have the same embedding dimension."""

    def __init__(self, num_dense_features: int, embedding_bag_collection: EmbeddingBagCollection, hidden_layer_size: int, deep_fm_dimension: int) -> None:
        super().__init__()
        configs = embedding_bag_collection.embedding_bag_configs()
        assert len(configs) > 0, "At least one embedding bag is required"
        embedding_dim: int = configs[0].embedding_dim
        assert all(c.embedding_dim == embedding_dim for c in configs), "All EmbeddingBagConfigs must have the same dimension"
        feature_names = [f for c in configs for f in c.feature_names]
        fm_in_features = embedding_dim * (1 + len(feature_names))
        self.sparse_arch = SparseArch(embedding_bag_collection)
        self.dense_arch = DenseArch(in_features=num_dense_features, hidden_layer_size=hidden_layer_size, embedding_dim=embedding_dim)
        self.inter_arch = FMInteractionArch(fm_in_features=fm_in_features, sparse_feature_names=feature_names, deep_fm_dimension=deep_fm_dimension)
        self.over_arch = OverArch(embedding_dim + deep_fm_dimension + 1)

    def forward(self, dense_features: torch.Tensor, sparse_features: KeyedJaggedTensor) -> torch.Tensor:
        embedded_dense = self.dense_arch(dense_features)
        embedded_sparse = self.sparse_arch(sparse_features)
        return self.over_arch(self.inter_arch(dense_features=embedded_dense, sparse_features=embedded_sparse))


class SimpleDeepFMNNWrapper(SimpleDeepFMNN):
    """Takes a batch object with ``float_features`` / ``idlist_features`` / ``label``; in training mode returns ``(loss, prediction)``,
    in eval mode the prediction."""

    def forward(self, model_input) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:  # type: ignore[override]
        pred = super().forward(model_input.float_features, model_input.idlist_features)
        if not self.training:
            return pred
        # the over arch ends in a sigmoid, so the loss is taken on probabilities
        loss = torch.nn.functional.binary_cross_entropy(pred.squeeze(-1), model_input.label.to(pred.dtype))
        return loss, pred
