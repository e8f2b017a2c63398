"""Position weighting for a group of features on one rank: every id gets the learned weight of its position inside its bag.

All features are served by one gather: the per-feature weight vectors are concatenated (so autograd splits the gradient back),
and each id indexes ``base[feature] + position``.  Positions come from the KJT's weights when the input dist already carried them
(row-wise sharding bucketizes positions with the ids), else from the offsets.
Counterpart of ``torchrec/distributed/grouped_position_weighted.py:22-120``."""
from __future__ import annotations

from collections import OrderedDict
from typing import Any, Dict, Iterator, Optional, Tuple

import torch
from torch import nn

from torchrec_b200.distributed.embedding_types import BaseGroupedFeatureProcessor
from torchrec_b200.ops import sparse_ops
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class GroupedPositionWeightedModule(BaseGroupedFeatureProcessor):
    def __init__(self, max_feature_lengths: Dict[str, int], device: Optional[torch.device] = None) -> None:
        super().__init__()
        if any(length <= 0 for length in max_feature_lengths.values()):
            raise ValueError(f"max feature lengths must be positive: {max_feature_lengths}")
        self.max_feature_lengths = max_feature_lengths
        self.position_weights: nn.ParameterDict = nn.ParameterDict(
            {key: nn.Parameter(torch.ones(length, device=device)) for key, length in max_feature_lengths.items()})

    def forward(self, features: KeyedJaggedTensor) -> KeyedJaggedTensor:
        values = features.values()
        if features.weights_or_none() is None:
            positions = sparse_ops.offsets_range(features.offsets().long(), values.numel())
        else:
            positions = features.weights().long()
        # one table = [1.0 (for features without weights)] ++ weights of every weighted feature present
        pieces = [torch.ones(1, device=values.device, dtype=torch.float32)]
        base, limit, cursor = [], [], 1
        for key in features.keys():
            if key in self.position_weights:
                w = self.position_weights[key]
                pieces.append(w)
                base.append(cursor)
                limit.append(w.numel() - 1)
                cursor += w.numel()
            else:
                base.append(0)
                limit.append(0)
        lpk = torch.tensor(features.length_per_key(), device=values.device)
        base_t = torch.repeat_interleave(torch.tensor(base, device=values.device), lpk, output_size=values.numel())
        limit_t = torch.repeat_interleave(torch.tensor(limit, device=values.device), lpk, output_size=values.numel())
        weights = torch.cat(pieces).index_select(0, base_t + torch.minimum(positions, limit_t))
        return KeyedJaggedTensor(
            keys=features.keys(), values=values, weights=weights, lengths=features.lengths(), offsets=features.offsets(),
            stride=features.stride(), length_per_key=features.length_per_key(),
            stride_per_key_per_rank=features.stride_per_key_per_rank() if features.variable_stride_per_key() else None)

    # only the position weights are state: the module has no buffers
    def named_parameters(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True) -> Iterator[Tuple[str, nn.Parameter]]:
        for name, param in self.position_weights.items():
            yield (f"{prefix}.position_weights.{name}" if prefix else f"position_weights.{name}"), param

    def named_buffers(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True) -> Iterator[Tuple[str, torch.Tensor]]:
        yield from ()

    def state_dict(self, destination: Optional[Dict[str, Any]] = None, prefix: str = "", keep_vars: bool = False) -> Dict[str, Any]:
        if destination is None:
            destination = OrderedDict()
            destination._metadata = OrderedDict()  # type: ignore[attr-defined]
        for name, param in self.position_weights.items():
            destination[f"{prefix}position_weights.{name}"] = param if keep_vars else param.detach()
        return destination
