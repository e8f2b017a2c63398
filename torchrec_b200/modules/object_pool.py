"""Base of the object pools: id-addressed storage that models read with ``lookup`` and write with ``update``
(``torchrec/modules/object_pool.py``)."""
from __future__ import annotations

import abc
from typing import Generic, TypeVar

import torch
from torch import nn

T = TypeVar("T")


class ObjectPool(abc.ABC, nn.Module, Generic[T]):
    @abc.abstractmethod
    def lookup(self, ids: torch.Tensor) -> T:
        ...

    @abc.abstractmethod
    def update(self, ids: torch.Tensor, values: T) -> None:
        ...
