"""DeepFM building blocks (counterpart of ``torchrec/modules/deepfm.py:36-215``)."""
from __future__ import annotations

from typing import List

import torch
from torch import nn


def _get_flatten_input(inputs: List[torch.Tensor]) -> torch.Tensor:
    return torch.cat([i.flatten(1) for i in inputs], dim=1)


class DeepFM(nn.Module):
    """Applies ``dense_module`` to the flattened concatenation of the embeddings."""

    def __init__(self, dense_module: nn.Module) -> None:
        super().__init__()
        self.dense_module = dense_module

    def forward(self, embeddings: List[torch.Tensor]) -> torch.Tensor:
        return self.dense_module(_get_flatten_input(embeddings))


class FactorizationMachine(nn.Module):
    """Second-order FM term ``0.5 * sum((sum x)^2 - sum x^2)`` -> ``[B, 1]``."""

    def __init__(self) -> None:
        super().__init__()

    def forward(self, embeddings: List[torch.Tensor]) -> torch.Tensor:
        fm_input = _get_flatten_input(embeddings)
        sum_of_input = torch.sum(fm_input, dim=1, keepdim=True)
        sum_of_square = torch.sum(fm_input * fm_input, dim=1, keepdim=True)
        square_of_sum = sum_of_input * sum_of_input
        cross_term = square_of_sum - sum_of_square
        return torch.sum(cross_term, dim=1, keepdim=True) * 0.5
