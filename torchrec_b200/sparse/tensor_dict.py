"""Adaptor from a ``tensordict.TensorDict`` of jagged entries to a ``KeyedJaggedTensor`` (``torchrec/sparse/tensor_dict.py:18``).
``tensordict`` is optional: without it only plain ``dict`` inputs are handled."""
from __future__ import annotations

from typing import Any, List, Optional

import torch

from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor

try:  # pragma: no cover - optional dependency
    from tensordict import TensorDict  # type: ignore
except Exception:  # pragma: no cover
    TensorDict = None  # type: ignore


def maybe_td_to_kjt(features: Any, keys: Optional[List[str]] = None) -> KeyedJaggedTensor:
    """Pass a KJT through; convert a TensorDict / dict ``{key: JaggedTensor | (values, lengths)}`` into a KJT."""
    if isinstance(features, KeyedJaggedTensor):
        return features
    is_td = TensorDict is not None and isinstance(features, TensorDict)
    if not is_td and not isinstance(features, dict):
        raise TypeError(f"expected KeyedJaggedTensor, TensorDict or dict, got {type(features).__name__}")
    if keys is None:
        keys = list(features.keys())
    values, lengths = [], []
    for k in keys:
        item = features[k]
        if isinstance(item, JaggedTensor):
            values.append(item.values()); lengths.append(item.lengths())
        elif isinstance(item, (tuple, list)) and len(item) == 2:
            values.append(item[0]); lengths.append(item[1])
        elif hasattr(item, "_values") and hasattr(item, "_offsets"):  # nested jagged tensor
            values.append(item._values); lengths.append(torch.diff(item._offsets))
        else:
            raise TypeError(f"entry {k} must be a JaggedTensor, a (values, lengths) pair or a nested jagged tensor")
    return KeyedJaggedTensor(keys=keys, values=torch.cat(values, dim=0), lengths=torch.cat(lengths, dim=0))
