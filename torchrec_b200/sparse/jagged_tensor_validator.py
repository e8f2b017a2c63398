"""Consistency checks for a ``KeyedJaggedTensor`` built from untrusted data (``torchrec/sparse/jagged_tensor_validator.py:14-123``).

The checks are a table of ``(predicate, message)`` rules evaluated in order; the first violated rule raises ``ValueError``
with the same wording as the reference, so callers that match on the text keep working.
"""
from __future__ import annotations

from typing import Callable, Iterator, List, Optional, Tuple

import torch

from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

Rule = Tuple[bool, Callable[[], str]]


def _first_violation(rules: Iterator[Rule]) -> None:
    for broken, message in rules:
        if broken:
            raise ValueError(message())


def _length_rules(lengths: torch.Tensor, n_values: int) -> Iterator[Rule]:
    total = int(lengths.sum())
    yield total != n_values, lambda: f"Sum of lengths must equal the number of values, but got {total} and {n_values}"
    yield bool((lengths < 0).any()), lambda: "lengths must be non-negative"


def _offset_rules(offsets: torch.Tensor, n_values: int) -> Iterator[Rule]:
    yield offsets.numel() == 0, lambda: "offsets cannot be empty"
    if offsets.numel() == 0:
        return
    first, last = int(offsets[0]), int(offsets[-1])
    yield first != 0, lambda: f"Expected first offset to be 0, but got {first}"
    yield last != n_values, lambda: f"The last element of offsets must equal to the number of values, but got {last} and {n_values}"
    yield bool((offsets[1:] < offsets[:-1]).any()), lambda: "offsets must be non-decreasing"


def _agreement_rules(lengths: torch.Tensor, offsets: torch.Tensor) -> Iterator[Rule]:
    nl, no = lengths.numel(), offsets.numel()
    yield nl != no - 1, lambda: f"Expected lengths size to be 1 more than offsets size, but got lengths size: {nl}, offsets size: {no}"
    if nl == no - 1:
        yield not torch.equal(lengths, offsets[1:] - offsets[:-1]), lambda: "offsets is not equal to the cumulative sum of lengths"


def _validate_lengths_and_offsets(kjt: KeyedJaggedTensor) -> None:
    lengths, offsets, n = kjt.lengths_or_none(), kjt.offsets_or_none(), kjt.values().numel()
    if lengths is None and offsets is None:
        raise ValueError("lengths and offsets cannot be both empty")
    if lengths is not None:
        _first_violation(_length_rules(lengths, n))
    if offsets is not None:
        _first_violation(_offset_rules(offsets, n))
    if lengths is not None and offsets is not None:
        _first_violation(_agreement_rules(lengths, offsets))


def _validate_lengths(lengths: torch.Tensor, values: torch.Tensor) -> None:
    _first_violation(_length_rules(lengths, values.numel()))


def _validate_offsets(offsets: torch.Tensor, values: torch.Tensor) -> None:
    _first_violation(_offset_rules(offsets, values.numel()))


def _bag_count(kjt: KeyedJaggedTensor) -> Optional[Tuple[str, int]]:
    lengths, offsets = kjt.lengths_or_none(), kjt.offsets_or_none()
    if lengths is not None:
        return "lengths size", lengths.numel()
    if offsets is not None:
        return "(offsets size - 1)", offsets.numel() - 1
    return None


def _validate_keys(kjt: KeyedJaggedTensor) -> None:
    keys: List[str] = kjt.keys()
    if len(keys) != len(set(keys)):
        raise ValueError(f"keys must be unique, but got {keys}")
    if not keys:
        if kjt.values().numel() != 0:
            raise ValueError("a KeyedJaggedTensor without keys cannot hold values")
        return
    counted = _bag_count(kjt)
    if counted is not None and not kjt.variable_stride_per_key():
        what, bags = counted
        if bags % len(keys) != 0:
            shown = bags if what == "lengths size" else bags + 1
            raise ValueError(f"{what} must be divisible by keys size, but got {shown} and {len(keys)}")


def _validate_weights(kjt: KeyedJaggedTensor) -> None:
    weights = kjt.weights_or_none()
    if weights is None:
        return
    n = kjt.values().numel()
    if weights.numel() != n:
        raise ValueError(f"weights size must equal to values size, but got {weights.numel()} and {n}")


def validate_keyed_jagged_tensor(kjt: KeyedJaggedTensor) -> None:
    """Raises ``ValueError`` when lengths / offsets / values / weights / keys disagree."""
    for check in (_validate_lengths_and_offsets, _validate_keys, _validate_weights):
        check(kjt)
