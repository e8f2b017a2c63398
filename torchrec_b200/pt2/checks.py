"""Guards used where code must behave differently under a graph-capturing tracer (``torchrec/pt2/checks.py:19-98``).  The hot
path of this framework is explicit kernels, streams and graphs, not a tracing compiler; the helpers exist so that models written
against them (and ``torch.export`` of the dense part) keep working."""
from __future__ import annotations

from typing import List

import torch

USE_TORCHDYNAMO_COMPILING_PATH: bool = False


def set_use_torchdynamo_compiling_path(val: bool) -> None:
    global USE_TORCHDYNAMO_COMPILING_PATH
    USE_TORCHDYNAMO_COMPILING_PATH = val


def get_use_torchdynamo_compiling_path() -> bool:
    return USE_TORCHDYNAMO_COMPILING_PATH


def is_torchdynamo_compiling() -> bool:
    if torch.jit.is_scripting():
        return False
    try:
        return get_use_torchdynamo_compiling_path() or torch.compiler.is_compiling()
    except Exception:
        return False


def is_non_strict_exporting() -> bool:
    try:
        from torch.compiler import is_exporting

        return bool(is_exporting())
    except Exception:
        return False


def is_pt2_compiling() -> bool:
    return is_torchdynamo_compiling() or is_non_strict_exporting()


def pt2_checks_tensor_slice(tensor: torch.Tensor, start_offset: int, end_offset: int, dim: int = 0) -> None:
    if torch.jit.is_scripting() or not is_pt2_compiling():
        return
    torch._check_is_size(start_offset)
    torch._check_is_size(end_offset)
    torch._check_is_size(end_offset - start_offset)
    torch._check(start_offset <= tensor.size(dim))
    torch._check(end_offset <= tensor.size(dim))
    torch._check(end_offset >= start_offset)


def pt2_checks_all_is_size(x: List[int]) -> List[int]:
    if torch.jit.is_scripting() or not is_pt2_compiling():
        return x
    for i in x:
        torch._check_is_size(i)
    return x


def pt2_check_size_nonzero(x: torch.Tensor) -> torch.Tensor:
    if torch.jit.is_scripting() or not is_pt2_compiling():
        return x
    for i in range(x.dim()):
        torch._check(x.size(i) > 0)
    return x


def pt2_guard_size_oblivious(x: bool) -> bool:
    if torch.jit.is_scripting() or not is_pt2_compiling():
        return x
    try:
        from torch.fx.experimental.symbolic_shapes import guard_size_oblivious

        return guard_size_oblivious(x)
    except Exception:
        return x
