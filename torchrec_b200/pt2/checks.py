"""Helpers for code that must behave differently while a graph-capturing tracer (dynamo, non-strict export) runs it.

The hot path of this framework is explicit kernels, streams and CUDA graphs, not a tracing compiler; these helpers exist so that
models written against them, and ``torch.export`` of the dense part, keep working.  Outside of tracing every helper is the identity.
Same surface as ``torchrec/pt2/checks.py:19-98``.
"""
from __future__ import annotations

from typing import Callable, List, TypeVar

import torch

T = TypeVar("T")
_force_compiling_path = False


def set_use_torchdynamo_compiling_path(val: bool) -> None:
    """Force the "being compiled" answer (for tests of the compile-only branches)."""
    global _force_compiling_path
    _force_compiling_path = bool(val)


def get_use_torchdynamo_compiling_path() -> bool:
    return _force_compiling_path


def _query(fn: Callable[[], bool]) -> bool:
    try:
        return bool(fn())
    except Exception:
        return False


def is_torchdynamo_compiling() -> bool:
    if torch.jit.is_scripting():
        return False
    return _force_compiling_path or _query(torch.compiler.is_compiling)


def is_non_strict_exporting() -> bool:
    return _query(lambda: torch.compiler.is_exporting())


def is_pt2_compiling() -> bool:
    return is_torchdynamo_compiling() or is_non_strict_exporting()


def _only_when_tracing(check: Callable[[T], None]) -> Callable[[T], T]:
    """``f(x) -> x`` that runs ``check(x)`` only under a tracer (and never under TorchScript)."""

    def wrapped(x: T) -> T:
        if not torch.jit.is_scripting() and is_pt2_compiling():
            check(x)
        return x

    return wrapped


def _all_sizes(xs: List[int]) -> None:
    for v in xs:
        torch._check_is_size(v)


def _nonzero_dims(t: torch.Tensor) -> None:
    for d in range(t.dim()):
        torch._check(t.size(d) > 0)


pt2_checks_all_is_size: Callable[[List[int]], List[int]] = _only_when_tracing(_all_sizes)
pt2_check_size_nonzero: Callable[[torch.Tensor], torch.Tensor] = _only_when_tracing(_nonzero_dims)


def pt2_checks_tensor_slice(tensor: torch.Tensor, start_offset: int, end_offset: int, dim: int = 0) -> None:
    """Tell the tracer that ``tensor[start:end]`` along ``dim`` is a valid, possibly empty, slice."""
    if torch.jit.is_scripting() or not is_pt2_compiling():
        return
    for v in (start_offset, end_offset, end_offset - start_offset):
        torch._check_is_size(v)
    n = tensor.size(dim)
    torch._check(start_offset <= n)
    torch._check(end_offset <= n)
    torch._check(start_offset <= end_offset)


def pt2_guard_size_oblivious(x: bool) -> bool:
    if torch.jit.is_scripting() or not is_pt2_compiling():
        return x
    try:
        from torch.fx.experimental.symbolic_shapes import guard_size_oblivious

        return guard_size_oblivious(x)
    except Exception:
        return x
