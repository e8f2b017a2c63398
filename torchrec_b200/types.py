"""Framework-wide small types (counterpart of ``torchrec/types.py:17-72``)."""
from __future__ import annotations

from abc import abstractmethod
from enum import Enum, unique

import torch
from torch import nn


class CacheMixin:
    """Modules that memoise per-batch computation expose ``clear_cache``."""

    @abstractmethod
    def clear_cache(self) -> None:
        ...


class CopyMixIn:
    @abstractmethod
    def copy(self, device: torch.device) -> nn.Module:
        ...


class ModuleCopyMixin(CopyMixIn):
    """``DistributedModelParallel`` copies the module to the target device."""

    def copy(self, device: torch.device) -> nn.Module:
        return self.to(device)  # type: ignore[attr-defined]


class ModuleNoCopyMixin(CopyMixIn):
    """``DistributedModelParallel`` leaves the module where it is."""

    def copy(self, device: torch.device) -> nn.Module:
        return self  # type: ignore[return-value]


@unique
class DataType(Enum):
    """Storage types an embedding table can use."""

    FP32 = "FP32"
    FP16 = "FP16"
    BF16 = "BF16"
    INT64 = "INT64"
    INT32 = "INT32"
    INT8 = "INT8"
    UINT8 = "UINT8"
    INT4 = "INT4"
    INT2 = "INT2"
    NFP8 = "NFP8"

    def __str__(self) -> str:
        return self.value
