"""Consistency checks for a ``KeyedJaggedTensor`` built from untrusted data (``torchrec/sparse/jagged_tensor_validator.py:14-123``)."""
from __future__ import annotations

import torch

from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


def validate_keyed_jagged_tensor(kjt: KeyedJaggedTensor) -> None:
    """Raises ``ValueError`` when lengths / offsets / values / weights / keys disagree."""
    _validate_lengths_and_offsets(kjt)
    _validate_keys(kjt)
    _validate_weights(kjt)


def _validate_lengths_and_offsets(kjt: KeyedJaggedTensor) -> None:
    lengths, offsets = kjt.lengths_or_none(), kjt.offsets_or_none()
    if lengths is None and offsets is None:
        raise ValueError("lengths and offsets cannot be both empty")
    if lengths is not None:
        _validate_lengths(lengths, kjt.values())
    if offsets is not None:
        _validate_offsets(offsets, kjt.values())
    if lengths is not None and offsets is not None:
        if lengths.numel() != offsets.numel() - 1:
            raise ValueError(f"Expected lengths size to be 1 more than offsets size, but got lengths size: {lengths.numel()}, offsets size: {offsets.numel()}")
        if not lengths.equal(torch.diff(offsets)):
            raise ValueError("offsets is not equal to the cumulative sum of lengths")


def _validate_lengths(lengths: torch.Tensor, values: torch.Tensor) -> None:
    if lengths.sum().item() != values.numel():
        raise ValueError(f"Sum of lengths must equal the number of values, but got {lengths.sum().item()} and {values.numel()}")
    if (lengths < 0).any():
        raise ValueError("lengths must be non-negative")


def _validate_offsets(offsets: torch.Tensor, values: torch.Tensor) -> None:
    if offsets.numel() == 0:
        raise ValueError("offsets cannot be empty")
    if offsets[0] != 0:
        raise ValueError(f"Expected first offset to be 0, but got {offsets[0]}")
    if offsets[-1] != values.numel():
        raise ValueError(f"The last element of offsets must equal to the number of values, but got {offsets[-1]} and {values.numel()}")
    if (torch.diff(offsets) < 0).any():
        raise ValueError("offsets must be non-decreasing")


def _validate_keys(kjt: KeyedJaggedTensor) -> None:
    keys = kjt.keys()
    if len(set(keys)) != len(keys):
        raise ValueError(f"keys must be unique, but got {keys}")
    lengths, offsets = kjt.lengths_or_none(), kjt.offsets_or_none()
    if lengths is not None and len(keys) > 0:
        if lengths.numel() % len(keys) != 0 and not kjt.variable_stride_per_key():
            raise ValueError(f"lengths size must be divisible by keys size, but got {lengths.numel()} and {len(keys)}")
    elif offsets is not None and len(keys) > 0:
        if (offsets.numel() - 1) % len(keys) != 0 and not kjt.variable_stride_per_key():
            raise ValueError(f"(offsets size - 1) must be divisible by keys size, but got {offsets.numel()} and {len(keys)}")
    if len(keys) == 0 and kjt.values().numel() != 0:
        raise ValueError("a KeyedJaggedTensor without keys cannot hold values")


def _validate_weights(kjt: KeyedJaggedTensor) -> None:
    weights = kjt.weights_or_none()
    if weights is not None and weights.numel() != kjt.values().numel():
        raise ValueError(f"weights size must equal to values size, but got {weights.numel()} and {kjt.values().numel()}")
