"""Feature processors: modules that rewrite the per-id weights of a KJT before the lookup.

``PositionWeightedModule`` gives the i-th id of every bag the learned weight ``position_weight[i]``;
``PositionWeightedModuleCollection`` does so for many features at once with one gather
(``torchrec/modules/feature_processor_.py:57,163``)."""
from __future__ import annotations

import abc
from typing import Dict, Iterator, List, Optional, Tuple

import torch
from torch import nn

from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor


def offsets_to_range_traceble(offsets: torch.Tensor, values: torch.Tensor) -> torch.Tensor:
    """Position of every value inside its bag: ``[0..l0-1, 0..l1-1, ...]``."""
    lengths = offsets[1:] - offsets[:-1]
    starts = torch.repeat_interleave(offsets[:-1], lengths, output_size=values.numel())
    return torch.arange(values.numel(), device=values.device, dtype=offsets.dtype) - starts


class FeatureProcessor(nn.Module):
    """Processes one feature's ``JaggedTensor``."""

    @abc.abstractmethod
    def forward(self, features: JaggedTensor) -> JaggedTensor:
        ...


class FeatureProcessorsCollection(nn.Module):
    """Processes a whole ``KeyedJaggedTensor``."""

    @abc.abstractmethod
    def forward(self, features: KeyedJaggedTensor) -> KeyedJaggedTensor:
        ...


class PositionWeightedModule(FeatureProcessor):
    def __init__(self, max_feature_length: int, device: Optional[torch.device] = None) -> None:
        super().__init__()
        self.position_weight = nn.Parameter(torch.empty([max_feature_length], device=device))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        with torch.no_grad():
            self.position_weight.fill_(1.0)

    def forward(self, features: JaggedTensor) -> JaggedTensor:
        seq = offsets_to_range_traceble(features.offsets(), features.values())
        weighted = torch.gather(self.position_weight, 0, seq.long())
        return JaggedTensor(values=features.values(), weights=weighted, lengths=features.lengths(), offsets=features.offsets())


def get_weights_list(cat_seq: torch.Tensor, features: KeyedJaggedTensor, position_weights: Dict[str, nn.Parameter]) -> Optional[torch.Tensor]:
    """Weight of every id of ``features`` given its position ``cat_seq`` inside its bag: the feature's position weight where the
    feature has one, 1 elsewhere.  The per-feature form of what ``PositionWeightedModuleCollection.forward`` does in one gather
    (``torchrec/modules/feature_processor_.py:139-153``)."""
    pieces = []
    for key, seq in zip(features.keys(), torch.split(cat_seq, features.length_per_key())):
        if key in position_weights:
            pieces.append(torch.gather(position_weights[key], 0, seq.long()))
        else:
            pieces.append(torch.ones(seq.shape[0], device=features.values().device))
    return torch.cat(pieces) if pieces else features.weights_or_none()


def get_stride_per_key_per_rank(kjt: KeyedJaggedTensor) -> Optional[List[List[int]]]:
    """The per-key per-rank batch sizes of a variable-batch KJT, None for a fixed batch."""
    return kjt.stride_per_key_per_rank() if kjt.variable_stride_per_key() else None


class PositionWeightedModuleCollection(FeatureProcessorsCollection):
    def __init__(self, max_feature_lengths: Dict[str, int], device: Optional[torch.device] = None) -> None:
        super().__init__()
        self.max_feature_lengths = max_feature_lengths
        for length in max_feature_lengths.values():
            if length <= 0:
                raise ValueError("max_feature_length must be positive")
        self.position_weights = nn.ParameterDict()
        self.position_weights_dict: Dict[str, nn.Parameter] = {}
        for key, length in max_feature_lengths.items():
            self.position_weights[key] = nn.Parameter(torch.empty([length], device=device))
            self.position_weights_dict[key] = self.position_weights[key]
        self.reset_parameters()

    def reset_parameters(self) -> None:
        with torch.no_grad():
            for key in self.max_feature_lengths:
                self.position_weights[key].fill_(1.0)
                self.position_weights_dict[key] = self.position_weights[key]

    def forward(self, features: KeyedJaggedTensor) -> KeyedJaggedTensor:
        """One concatenated weight vector, one gather: index = position in bag + start of the feature's weights."""
        keys = features.keys()
        cat_w = torch.cat([self.position_weights[k] for k in keys])
        starts, acc = [], 0
        for k in keys:
            starts.append(acc)
            acc += self.max_feature_lengths[k]
        # after a row-wise input distribution the bags are split and the position of every id inside its original bag travels
        # in the weights (torchrec/modules/feature_processor_.py:163 does the same)
        seq = offsets_to_range_traceble(features.offsets(), features.values()) if features.weights_or_none() is None else features.weights().long()
        lpk = torch.tensor(features.length_per_key(), device=features.values().device)
        base = torch.repeat_interleave(torch.tensor(starts, device=features.values().device), lpk, output_size=features.values().numel())
        weights = torch.gather(cat_w, 0, (seq.long() + base))
        return KeyedJaggedTensor(keys=keys, values=features.values(), weights=weights, lengths=features.lengths(), offsets=features.offsets(),
                                 stride=features.stride(), length_per_key=features.length_per_key())

    def copy(self, device: torch.device) -> nn.Module:
        self.position_weights = self.position_weights.to(device=device)
        for k in self.position_weights.keys():
            self.position_weights_dict[k] = self.position_weights[k]
        return self

    def _apply(self, *args, **kwargs):
        super()._apply(*args, **kwargs)
        for k, p in self.position_weights.items():
            self.position_weights_dict[k] = p
        return self
