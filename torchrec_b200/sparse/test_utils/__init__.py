"""Comparison helper for sparse types in tests (``torchrec/sparse/test_utils/__init__.py:17-90``)."""
from __future__ import annotations

from typing import Optional

import torch

from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


def _bagwise_sorted(t: torch.Tensor, lengths: torch.Tensor) -> torch.Tensor:
    """Sort the entries of every bag (order inside a pooled bag carries no meaning)."""
    seg = torch.repeat_interleave(torch.arange(lengths.numel(), device=t.device), lengths.long())
    by_value = torch.argsort(t, stable=True)
    return t[by_value[torch.argsort(seg[by_value], stable=True)]]


def _tensor_eq_or_none(t1: Optional[torch.Tensor], t2: Optional[torch.Tensor], out_of_order: bool = False, length: Optional[torch.Tensor] = None) -> bool:
    if t1 is None or t2 is None:
        return t1 is None and t2 is None
    if t1.dtype != t2.dtype or t1.shape != t2.shape:
        return False
    if not out_of_order:
        return torch.equal(t1, t2)
    assert length is not None
    a, b = _bagwise_sorted(t1, length), _bagwise_sorted(t2, length)
    return torch.allclose(a, b, rtol=1e-6, atol=1e-6) if torch.is_floating_point(a) else torch.equal(a, b)


def keyed_jagged_tensor_equals(kjt1: Optional[KeyedJaggedTensor], kjt2: Optional[KeyedJaggedTensor], is_pooled_features: bool = False) -> bool:
    """Same keys, lengths, values and weights; with ``is_pooled_features`` the order of the ids inside a bag is ignored."""
    if kjt1 is None or kjt2 is None:
        return kjt1 is None and kjt2 is None
    if kjt1.keys() != kjt2.keys() or not _tensor_eq_or_none(kjt1.lengths(), kjt2.lengths()):
        return False
    return (_tensor_eq_or_none(kjt1.values(), kjt2.values(), is_pooled_features, kjt1.lengths())
            and _tensor_eq_or_none(kjt1.weights_or_none(), kjt2.weights_or_none(), is_pooled_features, kjt1.lengths()))
