"""What a serializer of exportable modules has to provide.

``encapsulate_ir_modules`` / ``decapsulate_ir_modules`` (``ir/utils.py``) walk a model and, for every module whose qualified class name
is a key of ``module_to_serializer_cls``, hand the module to the serializer.  A serializer therefore decides three things: which
module types it understands, how such a module is frozen into metadata (``encapsulate_module``) and how it is rebuilt
(``decapsulate_module``).  ``ir/serializer.py`` has the JSON implementation.  Same contract as ``torchrec/ir/types.py:20``.
"""
from __future__ import annotations

import abc
from typing import Any, Dict, List, Optional

import torch
from torch import nn


class SerializerInterface(abc.ABC):
    #: qualified class name -> serializer class handling that module type
    module_to_serializer_cls: Dict[str, Any] = {}

    @classmethod
    @abc.abstractmethod
    def encapsulate_module(cls, module: nn.Module) -> List[str]:
        """Freeze ``module`` in place: store its metadata in an ``ir_metadata`` buffer and replace its forward by an opaque op.
        Returns the names of the children that still need a pass of their own."""
        raise NotImplementedError

    @classmethod
    @abc.abstractmethod
    def decapsulate_module(cls, module: nn.Module, device: Optional[torch.device] = None) -> nn.Module:
        """Build the real module again from the ``ir_metadata`` buffer found on ``module`` (an unflattened export)."""
        raise NotImplementedError

    @classmethod
    def handles(cls, module: nn.Module) -> bool:
        t = type(module)
        return f"{t.__module__}.{t.__qualname__}" in cls.module_to_serializer_cls
