"""Mixins for objects that cross CUDA streams or devices.

Mirrors the contracts of the reference's ``torchrec/streamable.py:15-48``: anything a
training pipeline moves between streams implements ``record_stream`` and anything it
copies to a device implements ``to``.
"""
from __future__ import annotations

import abc

import torch


class Multistreamable(abc.ABC):
    """Objects holding tensors that may be consumed on a stream other than the producer's."""

    @abc.abstractmethod
    def record_stream(self, stream: torch.Stream) -> None:
        ...


class Pipelineable(Multistreamable):
    """A batch (or part of one) that a train pipeline can copy to the device ahead of time."""

    @abc.abstractmethod
    def to(self, device: torch.device, non_blocking: bool = False) -> "Pipelineable":
        ...
