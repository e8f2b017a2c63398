"""Fused-optimizer interfaces (cf. ``torchrec/optim/fused.py:17-57``).

A fused optimizer updates its parameters inside the backward pass of the embedding kernel;
``step()`` and ``zero_grad()`` are therefore (almost) no-ops that exist so that training loops
can treat it like any other optimizer.
"""
from __future__ import annotations

import abc
from typing import Any

from torch import optim

from torchrec_b200.optim.keyed import KeyedOptimizer


class FusedOptimizer(KeyedOptimizer, abc.ABC):
    @abc.abstractmethod
    def step(self, closure: Any = None) -> None:
        ...

    @abc.abstractmethod
    def zero_grad(self, set_to_none: bool = False) -> None:
        ...

    def __repr__(self) -> str:
        return optim.Optimizer.__repr__(self)


class EmptyFusedOptimizer(FusedOptimizer):
    def __init__(self) -> None:
        super().__init__({}, {}, {})

    def step(self, closure: Any = None) -> None:
        pass

    def zero_grad(self, set_to_none: bool = False) -> None:
        pass


class FusedOptimizerModule(abc.ABC):
    """A module that owns a fused optimizer."""

    @property
    @abc.abstractmethod
    def fused_optimizer(self) -> KeyedOptimizer:
        ...
