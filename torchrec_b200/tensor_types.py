"""Sub-byte tensor views: ``UInt4Tensor`` / ``UInt2Tensor`` wrap a ``uint8`` tensor and present it with ``8 / bits`` times as
many elements along the last dimension, so quantized table rows can be sliced, viewed and moved in element units.

Supported through ``__torch_dispatch__``: ``detach``, ``clone``, ``copy_``, ``.view(torch.uint8)`` (the packed bytes),
``.to(device)``, ``slice`` (last-dim bounds must fall on byte boundaries), ``view(shape)`` and ``select`` on any dimension but the
last.  Anything else raises ``NotImplementedError``.  Counterpart of ``torchrec/tensor_types.py:20-180``."""
from __future__ import annotations

import itertools
from typing import Any, Callable, Dict, List, Sequence, Tuple

import torch
from torch._prims_common import infer_size

aten = torch.ops.aten


def down_size(N: int, size: Sequence[int]) -> Tuple[int, ...]:
    """Shape of the packed bytes for an element shape (``N`` elements per byte)."""
    assert size[-1] % N == 0, f"{tuple(size)} last dim not divisible by {N}"
    return (*size[:-1], size[-1] // N)


def up_size(N: int, size: Sequence[int]) -> Tuple[int, ...]:
    return (*size[:-1], size[-1] * N)


def fill_defaults(args: Sequence[Any], n: int, defaults_tail: Sequence[Any]) -> List[Any]:
    """Pad a dispatch argument list to ``n`` entries with the trailing defaults: ``fill_defaults([1, 2, 3], 5, [3, 4, 5])`` ->
    ``[1, 2, 3, 4, 5]``."""
    if n - len(defaults_tail) > len(args):
        raise RuntimeError("not enough defaults to fill arguments")
    return list(args) + list(defaults_tail[len(defaults_tail) - (n - len(args)):]) if n > len(args) else list(args)


def find_arg_of_type(it, t):
    return next((x for x in it if isinstance(x, t)), None)


class UIntXTensor(torch.Tensor):
    """``N`` elements per stored byte; reported dtype stays ``uint8`` and the reported last dim is ``N`` x the stored one."""

    __torch_function__ = torch._C._disabled_torch_function_impl

    @staticmethod
    def __new__(cls, N: int, elem: torch.Tensor):
        assert elem.dtype is torch.uint8
        return torch.Tensor._make_wrapper_subclass(cls, up_size(N, elem.shape), dtype=torch.uint8, device=elem.device)

    def __init__(self, N: int, elem: torch.Tensor) -> None:
        self.N: int = N
        self.elem: torch.Tensor = elem

    def tolist(self) -> List:
        return self.elem.tolist()

    def __repr__(self) -> str:
        return f"UInt{8 // self.N}Tensor(shape={tuple(self.shape)}, elem={self.elem})"

    # ---- op handlers: each gets (cls, args, kwargs) and returns the result or NotImplemented ---------------------------
    @staticmethod
    def _on_bytes(func):
        def run(cls, args, kwargs):
            return cls(func(args[0].elem))
        return run

    @staticmethod
    def _detach(cls, args, kwargs):
        with torch.inference_mode(False):
            return cls(aten.detach.default(args[0].elem))

    @staticmethod
    def _copy(cls, args, kwargs):
        dst, src = args[0], args[1]
        dst.elem.copy_(src.elem if isinstance(src, UIntXTensor) else src)
        return dst

    @staticmethod
    def _view_dtype(cls, args, kwargs):
        return args[0].elem if args[1] == torch.uint8 else NotImplemented

    @staticmethod
    def _to_copy(cls, args, kwargs):
        everything = list(itertools.chain(args, kwargs.values()))
        device = find_arg_of_type(everything, torch.device)
        dtype = find_arg_of_type(everything, torch.dtype)
        if device is None:
            return NotImplemented
        assert dtype is None or dtype == torch.uint8
        return cls(args[0].elem.to(device))

    @staticmethod
    def _slice(cls, args, kwargs):
        self, dim, start, end, step = fill_defaults(args, 5, [0, None, None, 1])
        dim = dim % self.dim()
        if dim != self.dim() - 1:
            return cls(aten.slice.Tensor(self.elem, dim, start, end, step))
        if step != 1:
            raise NotImplementedError(f"slice step={step}")
        start = 0 if start is None else start
        end = self.shape[dim] if end is None else min(end, self.shape[dim])
        assert start % self.N == 0 and end % self.N == 0, (start, end)
        return cls(aten.slice.Tensor(self.elem, dim, start // self.N, end // self.N, 1))

    @staticmethod
    def _view(cls, args, kwargs):
        self, size = args
        return cls(self.elem.reshape(down_size(self.N, infer_size(size, self.numel()))))

    @staticmethod
    def _select(cls, args, kwargs):
        self, dim, index = args
        if dim % self.dim() == self.dim() - 1:
            raise NotImplementedError("select along the packed dimension")
        return cls(aten.select.int(self.elem, dim, index))

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        handlers: Dict[Any, Callable] = {
            aten.detach.default: UIntXTensor._detach,
            aten.clone.default: UIntXTensor._on_bytes(aten.clone.default),
            aten.copy_.default: UIntXTensor._copy,
            aten.view.dtype: UIntXTensor._view_dtype,
            aten._to_copy.default: UIntXTensor._to_copy,
            aten.slice.Tensor: UIntXTensor._slice,
            aten.view.default: UIntXTensor._view,
            aten.select.int: UIntXTensor._select,
        }
        handler = handlers.get(func)
        out = handler(cls, args, kwargs or {}) if handler is not None else NotImplemented
        if out is NotImplemented:
            raise NotImplementedError(f"{func} args:{args} kwargs:{kwargs}")
        return out


class UInt4Tensor(UIntXTensor):
    """Two 4-bit elements per byte."""

    N: int = 2

    @staticmethod
    def __new__(cls, elem: torch.Tensor):
        return UIntXTensor.__new__(cls, cls.N, elem)

    def __init__(self, elem: torch.Tensor) -> None:
        UIntXTensor.__init__(self, UInt4Tensor.N, elem)


class UInt2Tensor(UIntXTensor):
    """Four 2-bit elements per byte."""

    N: int = 4

    @staticmethod
    def __new__(cls, elem: torch.Tensor):
        return UIntXTensor.__new__(cls, cls.N, elem)

    def __init__(self, elem: torch.Tensor) -> None:
        UIntXTensor.__init__(self, UInt2Tensor.N, elem)
