"""Input shaping for traced / exported models (``torchrec/pt2/utils.py:28-185``)."""
from __future__ import annotations

import functools
from typing import Any, Callable, List, Optional, Tuple

import torch

from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


def kjt_for_pt2_tracing(kjt: KeyedJaggedTensor, convert_to_vb: bool = False, mark_length: bool = False) -> KeyedJaggedTensor:
    """A copy of ``kjt`` in the form a tracer handles best: int64 lengths, offsets dropped (recomputed inside the graph), the
    value dimension marked dynamic; optionally converted to the variable-batch layout with equal strides."""
    is_vb = kjt.variable_stride_per_key()
    if convert_to_vb and is_vb:
        return kjt
    n = len(kjt.keys())
    lengths = kjt.lengths().long()
    stride = kjt.stride()
    values = kjt.values().long()
    weights = kjt.weights_or_none()
    try:
        torch._dynamo.decorators.mark_unbacked(values, 0)
        if weights is not None:
            torch._dynamo.decorators.mark_unbacked(weights, 0)
        if mark_length:
            torch._dynamo.decorators.mark_dynamic(lengths, 0)
    except Exception:
        pass
    if convert_to_vb:
        spkpr = [[stride]] * n
        inv = torch.arange(stride, device=values.device).expand(n, stride).contiguous()
        return KeyedJaggedTensor(keys=kjt.keys(), values=values, weights=weights, lengths=lengths, stride_per_key_per_rank=spkpr, inverse_indices=(kjt.keys(), inv))
    return KeyedJaggedTensor(keys=kjt.keys(), values=values, weights=weights, lengths=lengths, stride=stride)


def default_pipeline_input_transformer(inp: Any) -> Any:
    """Apply :func:`kjt_for_pt2_tracing` to every KJT attribute of a batch object."""
    for name in ("id_list_features", "id_score_list_features", "sparse_features"):
        if hasattr(inp, name):
            attr = getattr(inp, name)
            if isinstance(attr, KeyedJaggedTensor):
                setattr(inp, name, kjt_for_pt2_tracing(attr))
    return inp


_FAKE_REGISTERED = False


def register_fake_classes() -> None:
    """Fake (shape-only) counterparts of the script classes of the native libraries, so that exporting a model that holds them does
    not run native code.  The only script classes here are the dynamic-embedding ones, which never sit inside an exported graph."""
    global _FAKE_REGISTERED
    _FAKE_REGISTERED = True


def deregister_fake_classes() -> None:
    global _FAKE_REGISTERED
    _FAKE_REGISTERED = False


def pt2_compile_callable(f: Callable) -> Callable:
    """Method decorator: compile ``f`` on first use when the owning object has ``_pt2_compile = True``."""

    @functools.wraps(f)
    def inner(self: Any, *args: Any, **kwargs: Any) -> Any:
        if getattr(self, "_pt2_compile", False):
            compiled = getattr(self, "_pt2_compiled_fn", None)
            if compiled is None:
                compiled = torch.compile(functools.partial(f, self), fullgraph=True, dynamic=True)
                self._pt2_compiled_fn = compiled
            return compiled(*args, **kwargs)
        return f(self, *args, **kwargs)

    return inner
