"""Mark parameters so that their optimizer runs inside the backward pass.

For embedding tables the mark (``_optimizer_classes`` / ``_optimizer_kwargs``) is what the
sharders read to choose the fused update of the TBE kernel
(cf. ``torchrec/optim/apply_optimizer_in_backward.py:16`` and
``torchrec/distributed/embeddingbag.py:673-692``).
"""
from __future__ import annotations

from typing import Any, Dict, Iterable, Type
from warnings import warn

import torch


def apply_optimizer_in_backward(
    optimizer_class: Type[torch.optim.Optimizer],
    params: Iterable[torch.nn.Parameter],
    optimizer_kwargs: Dict[str, Any],
) -> None:
    """Attach ``optimizer_class(**optimizer_kwargs)`` to every parameter in ``params``.

    Dense parameters get a gradient-accumulation hook that steps a private optimizer as soon
    as the gradient is ready and then frees it; embedding tables handled by a sharded module
    never materialise a gradient -- the kernel applies the update.
    """
    for param in params:
        if getattr(param, "_in_backward_optimizers", None):
            warn("apply_optimizer_in_backward was already called on this parameter; the new optimizer is added", stacklevel=2)
        else:
            param._in_backward_optimizers = []  # type: ignore[attr-defined]
            param._optimizer_classes = []  # type: ignore[attr-defined]
            param._optimizer_kwargs = []  # type: ignore[attr-defined]
        opt = optimizer_class([param], **optimizer_kwargs)
        param._in_backward_optimizers.append(opt)  # type: ignore[attr-defined]
        param._optimizer_classes.append(optimizer_class)  # type: ignore[attr-defined]
        param._optimizer_kwargs.append(optimizer_kwargs)  # type: ignore[attr-defined]
        if param.device.type == "meta" or not param.requires_grad:
            continue

        def _make_hook(p):
            def hook(*_unused):
                for o in p._in_backward_optimizers:
                    o.step()
                p.grad = None

            return hook

        if hasattr(param, "register_post_accumulate_grad_hook"):
            param._in_backward_hook = param.register_post_accumulate_grad_hook(_make_hook(param))  # type: ignore[attr-defined]
