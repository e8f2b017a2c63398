"""Interface of an IR serializer (``torchrec/ir/types.py:20``)."""
from __future__ import annotations

import abc
from typing import Any, Dict, List, Optional

import torch
from torch import nn


class SerializerInterface(abc.ABC):
    """Turns supported modules into (metadata buffer + opaque forward) and back."""

    @classmethod
    @property
    def module_to_serializer_cls(cls) -> Dict[str, Any]:
        raise NotImplementedError

    @classmethod
    @abc.abstractmethod
    def encapsulate_module(cls, module: nn.Module) -> List[str]:
        """Serialise ``module`` in place; returns the children that need their own pass."""

    @classmethod
    @abc.abstractmethod
    def decapsulate_module(cls, module: nn.Module, device: Optional[torch.device] = None) -> nn.Module:
        """Rebuild the original module from the ``ir_metadata`` buffer of ``module``."""
