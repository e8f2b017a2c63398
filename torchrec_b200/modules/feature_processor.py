"""Legacy grouped feature processors: one ``BaseFeatureProcessor`` per feature applied to a KJT by
``BaseGroupedFeatureProcessor`` (``torchrec/modules/feature_processor.py:54,124``)."""
from __future__ import annotations

import abc
from typing import Dict, Optional

import torch
from torch import nn

from torchrec_b200.modules.feature_processor_ import offsets_to_range_traceble
from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor


class BaseFeatureProcessor(nn.Module):
    @abc.abstractmethod
    def forward(self, features: Dict[str, JaggedTensor]) -> Dict[str, JaggedTensor]:
        ...


def position_weighted_module_update_features(features: Dict[str, JaggedTensor], weighted_features: Dict[str, JaggedTensor]) -> Dict[str, JaggedTensor]:
    """``features`` with the entries of ``weighted_features`` put in place of the unweighted ones (features without a position weight
    pass through)."""
    features.update(weighted_features)
    return features


class PositionWeightedModule(BaseFeatureProcessor):
    def __init__(self, max_feature_lengths: Dict[str, int], device: Optional[torch.device] = None) -> None:
        super().__init__()
        self.max_feature_lengths = max_feature_lengths
        self.position_weights = nn.ParameterDict({k: nn.Parameter(torch.ones(n, device=device)) for k, n in max_feature_lengths.items()})

    def forward(self, features: Dict[str, JaggedTensor]) -> Dict[str, JaggedTensor]:
        out: Dict[str, JaggedTensor] = {}
        for key, pw in self.position_weights.items():
            jt = features[key]
            seq = offsets_to_range_traceble(jt.offsets(), jt.values())
            out[key] = JaggedTensor(values=jt.values(), lengths=jt.lengths(), offsets=jt.offsets(), weights=torch.gather(pw, 0, seq.long()))
        return position_weighted_module_update_features(features, out)


class BaseGroupedFeatureProcessor(nn.Module):
    @abc.abstractmethod
    def forward(self, features: KeyedJaggedTensor) -> KeyedJaggedTensor:
        ...


class PositionWeightedProcessor(BaseGroupedFeatureProcessor):
    """Applies position weights to the listed features of a KJT (others get weight 1)."""

    def __init__(self, max_feature_lengths: Dict[str, int], device: Optional[torch.device] = None) -> None:
        super().__init__()
        self.max_feature_lengths = max_feature_lengths
        self.position_weights = nn.ParameterDict({k: nn.Parameter(torch.ones(n, device=device)) for k, n in max_feature_lengths.items()})

    def forward(self, features: KeyedJaggedTensor) -> KeyedJaggedTensor:
        seq = offsets_to_range_traceble(features.offsets(), features.values()).long()
        weights = torch.ones(features.values().numel(), device=features.values().device)
        start = 0
        for key, n in zip(features.keys(), features.length_per_key()):
            if key in self.position_weights:
                weights[start: start + n] = torch.gather(self.position_weights[key], 0, seq[start: start + n])
            start += n
        return KeyedJaggedTensor(keys=features.keys(), values=features.values(), weights=weights, lengths=features.lengths(), offsets=features.offsets(),
                                 stride=features.stride(), length_per_key=features.length_per_key())
