"""DLRM whose pairwise-dot interaction is replaced by a transformer encoder over the ``F + 1`` feature vectors
(``torchrec/models/experimental/transformerdlrm.py:18-200``)."""
from __future__ import annotations

from typing import List, Optional

import torch
from torch import nn

from torchrec_b200.models.dlrm import DLRM, OverArch
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection


class InteractionTransformerArch(nn.Module):
    """Self-attention over ``[dense, sparse_0, .., sparse_{F-1}]``: ``[B, D]`` and ``[B, F, D]`` -> ``[B, (F + 1) * D]``.

    The encoder layers are the sequence-first default, so attention runs along dim 0 of the ``[B, F + 1, D]`` stack exactly as
    in the counterpart; ``batch_first=True`` makes it attend over the features of one sample instead."""

    def __init__(self, num_sparse_features: int, embedding_dim: int, nhead: int = 8, ntransformer_layers: int = 4, batch_first: bool = False) -> None:
        super().__init__()
        self.F: int = num_sparse_features
        self.nhead = nhead
        self.ntransformer_layers = ntransformer_layers
        layer = nn.TransformerEncoderLayer(d_model=embedding_dim, nhead=nhead, batch_first=batch_first)
        self.interarch_TE = nn.TransformerEncoder(layer, num_layers=ntransformer_layers, enable_nested_tensor=False)

    def forward(self, dense_features: torch.Tensor, sparse_features: torch.Tensor) -> torch.Tensor:
        if self.F <= 0:
            return dense_features
        stacked = torch.cat((dense_features.unsqueeze(1), sparse_features), dim=1)
        return self.interarch_TE(stacked).reshape(dense_features.shape[0], -1)


class DLRM_Transformer(DLRM):
    """DLRM with ``InteractionTransformerArch``; the over arch sees ``(F + 1) * D`` features."""

    def __init__(self, embedding_bag_collection: EmbeddingBagCollection, dense_in_features: int, dense_arch_layer_sizes: List[int],
                 over_arch_layer_sizes: List[int], nhead: int = 8, ntransformer_layers: int = 4, dense_device: Optional[torch.device] = None) -> None:
        super().__init__(embedding_bag_collection, dense_in_features, dense_arch_layer_sizes, over_arch_layer_sizes, dense_device)
        embedding_dim: int = embedding_bag_collection.embedding_bag_configs()[0].embedding_dim
        num_sparse_features: int = len(self.sparse_arch.sparse_feature_names)
        self.inter_arch = InteractionTransformerArch(num_sparse_features, embedding_dim, nhead=nhead, ntransformer_layers=ntransformer_layers)
        if dense_device is not None:
            self.inter_arch = self.inter_arch.to(dense_device)
        self.over_arch = OverArch(in_features=(num_sparse_features + 1) * embedding_dim, layer_sizes=over_arch_layer_sizes, device=dense_device)
