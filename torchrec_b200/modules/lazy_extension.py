"""``LazyModuleExtensionMixin``: lazy modules whose first forward may receive keyword arguments, and ``lazy_apply`` to queue
functions (weight initialisers) that run right after the parameters materialise (``torchrec/modules/lazy_extension.py:43,103``)."""
from __future__ import annotations

import functools
import inspect
from typing import Any, Callable

import torch
from torch.nn.modules.lazy import LazyModuleMixin


def _apply_functions_after_first_forward(module: torch.nn.Module, input: Any, output: Any) -> None:
    for fn in getattr(module, "_functions_to_lazy_apply", None) or []:
        module.apply(fn)
    handle = getattr(module, "_lazy_apply_hook", None)
    if handle is not None:
        handle.remove()
    for name in ("_functions_to_lazy_apply", "_lazy_apply_hook"):
        if hasattr(module, name):
            delattr(module, name)


def lazy_apply(module: torch.nn.Module, fn: Callable[[torch.nn.Module], None]) -> torch.nn.Module:
    """Queue ``fn`` to be applied to ``module`` (and its children) after its first forward, when lazy parameters exist."""
    if not hasattr(module, "_functions_to_lazy_apply"):
        module._functions_to_lazy_apply = []  # type: ignore[assignment]
    if not hasattr(module, "_lazy_apply_hook"):
        module._lazy_apply_hook = module.register_forward_hook(_apply_functions_after_first_forward)  # type: ignore[assignment]
    module._functions_to_lazy_apply.append(fn)  # type: ignore[union-attr]
    return module


class LazyModuleExtensionMixin(LazyModuleMixin):
    """Differences to ``LazyModuleMixin``: ``initialize_parameters`` receives the keyword arguments of the first call too, and
    ``apply`` is refused while parameters are uninitialised (use ``lazy_apply``)."""

    def apply(self, fn: Callable[[torch.nn.Module], None]) -> torch.nn.Module:
        if hasattr(self, "_initialize_hook"):
            raise RuntimeError("Module {} has not been initialized. Call module.forward once, or use lazy_apply(module, fn).".format(self))
        return super().apply(fn)  # type: ignore[misc]

    def _infer_parameters(self, module, args, kwargs=None) -> None:  # type: ignore[override]
        kwargs = kwargs if kwargs is not None else {}
        module.initialize_parameters(*args, **kwargs)
        if module.has_uninitialized_params():
            raise RuntimeError(f"module {self._get_name()} has not been fully initialized")
        module._initialize_hook.remove()
        module._load_hook.remove()
        delattr(module, "_initialize_hook")
        delattr(module, "_load_hook")
        if module.cls_to_become is not None:
            module.__class__ = module.cls_to_become

    def __init__(self, *args: Any, **kwargs: Any) -> None:
        super().__init__(*args, **kwargs)
        # replace the positional-only hook of the base mixin by one that also sees keyword arguments
        self._initialize_hook.remove()  # type: ignore[has-type]
        self._initialize_hook = self.register_forward_pre_hook(self._infer_parameters, with_kwargs=True)  # type: ignore[attr-defined]
