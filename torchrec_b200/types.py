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


class _PackedIntTensor:
    """Logical ``[rows, cols]`` tensor of ``bits``-bit unsigned integers packed into a uint8 tensor ``[rows, cols * bits / 8]``
    (lowest bits first inside a byte).  Used for int4 / int2 embedding payloads in state dicts
    (``UInt4Tensor`` / ``UInt2Tensor`` of ``torchrec/types.py``)."""

    BITS = 8

    def __init__(self, packed: "torch.Tensor") -> None:
        import torch as _torch

        assert packed.dtype == _torch.uint8 and packed.dim() == 2
        self.elem = packed

    @property
    def shape(self):
        import torch as _torch

        return _torch.Size([self.elem.shape[0], self.elem.shape[1] * (8 // self.BITS)])

    def size(self, dim=None):
        return self.shape if dim is None else self.shape[dim]

    @property
    def device(self):
        return self.elem.device

    def to(self, *args, **kwargs):
        return type(self)(self.elem.to(*args, **kwargs))

    def detach(self):
        return type(self)(self.elem.detach())

    def clone(self):
        return type(self)(self.elem.clone())

    def unpack(self) -> "torch.Tensor":
        """uint8 ``[rows, cols]`` of the stored integers."""
        import torch as _torch

        per = 8 // self.BITS
        shifts = _torch.arange(per, device=self.elem.device, dtype=_torch.int32) * self.BITS
        return ((self.elem.to(_torch.int32).unsqueeze(-1) >> shifts) & (2 ** self.BITS - 1)).reshape(self.elem.shape[0], -1).to(_torch.uint8)

    @classmethod
    def pack(cls, values: "torch.Tensor") -> "_PackedIntTensor":
        import torch as _torch

        per = 8 // cls.BITS
        assert values.dim() == 2 and values.shape[1] % per == 0
        v = values.to(_torch.int32).view(values.shape[0], -1, per)
        shifts = _torch.arange(per, device=values.device, dtype=_torch.int32) * cls.BITS
        return cls((v << shifts).sum(-1).to(_torch.uint8))

    def __repr__(self) -> str:
        return f"{type(self).__name__}(shape={tuple(self.shape)})"


class UInt4Tensor(_PackedIntTensor):
    BITS = 4


class UInt2Tensor(_PackedIntTensor):
    BITS = 2
