"""Embedding towers: an embedding module together with the interaction that consumes only its output, so that a sharder can
place both on the same ranks and ship the (smaller) interaction output (``torchrec/modules/embedding_tower.py:39,88``)."""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
from torch import nn

from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection, EmbeddingCollection
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


def _check_module_type(m: nn.Module) -> None:
    if not isinstance(m, (EmbeddingBagCollection, EmbeddingCollection)):
        raise RuntimeError(f"tower embedding module must be an EmbeddingBagCollection or EmbeddingCollection, got {type(m).__name__}")


def tower_input_params(module: nn.Module) -> Tuple[bool, bool]:
    """``(has unweighted features, has weighted features)`` of the tower's embedding module."""
    if isinstance(module, EmbeddingCollection):
        return True, False
    return (not module.is_weighted(), module.is_weighted())


class EmbeddingTower(nn.Module):
    def __init__(self, embedding_module: nn.Module, interaction_module: nn.Module, device: Optional[torch.device] = None) -> None:
        super().__init__()
        _check_module_type(embedding_module)
        self.embedding = embedding_module
        self.interaction = interaction_module

    def forward(self, *args, **kwargs) -> torch.Tensor:
        return self.interaction(self.embedding(*args, **kwargs))


class EmbeddingTowerCollection(nn.Module):
    """Runs every tower on the features it needs and concatenates the tower outputs along dim 1."""

    def __init__(self, towers: List[EmbeddingTower], device: Optional[torch.device] = None) -> None:
        super().__init__()
        self.towers = nn.ModuleList(towers)
        self._input_params: List[Tuple[bool, bool]] = [tower_input_params(t.embedding) for t in towers]

    def forward(self, features: Optional[KeyedJaggedTensor] = None, weighted_features: Optional[KeyedJaggedTensor] = None) -> torch.Tensor:
        outs = []
        for tower, (has_f, has_w) in zip(self.towers, self._input_params):
            if has_f and has_w:
                outs.append(tower(features, weighted_features))
            elif has_f:
                outs.append(tower(features))
            else:
                outs.append(tower(weighted_features))
        return torch.cat(outs, dim=1)
