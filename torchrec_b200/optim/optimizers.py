"""Marker optimizer classes for ``apply_optimizer_in_backward`` on embedding tables.

``step`` is a no-op: only the class and its keyword arguments matter -- sharders translate
them into the fused update of the embedding kernel (cf. ``torchrec/optim/optimizers.py:20-181``,
mapping in ``torchrec/distributed/utils.py:330-354``).
"""
from __future__ import annotations

from typing import Any, Dict, Iterable, Iterator, Tuple

import torch
from torch import nn
from torch.optim.optimizer import Optimizer


def in_backward_optimizer_filter(named_parameters: Iterator[Tuple[str, nn.Parameter]], include: bool = False) -> Iterator[Tuple[str, nn.Parameter]]:
    """Keep (``include=True``) or drop (default) parameters whose optimizer runs in backward."""
    for fqn, param in named_parameters:
        if hasattr(param, "_in_backward_optimizers") == include:
            yield fqn, param


class _Marker(Optimizer):
    def step(self, closure: Any = None) -> None:  # type: ignore[override]
        pass


class SGD(_Marker):
    def __init__(self, params: Iterable[torch.nn.Parameter], lr: float = 1e-2, momentum: float = 0, weight_decay: float = 0, gradient_clipping: bool = False, max_gradient: float = 1.0) -> None:
        self._params = params
        super().__init__(params, {"lr": lr, "momentum": momentum, "weight_decay": weight_decay, "gradient_clipping": gradient_clipping, "max_gradient": max_gradient})


class LarsSGD(_Marker):
    def __init__(self, params, lr: float = 1e-2, momentum: float = 0, weight_decay: float = 0, eta: float = 0.001, gradient_clipping: bool = False, max_gradient: float = 1.0) -> None:
        self._params = params
        super().__init__(params, {"lr": lr, "momentum": momentum, "weight_decay": weight_decay, "eta": eta, "gradient_clipping": gradient_clipping, "max_gradient": max_gradient})


class LAMB(_Marker):
    def __init__(self, params, lr: float = 1e-2, betas: Tuple[float, float] = (0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0, gradient_clipping: bool = False, max_gradient: float = 1.0) -> None:
        self._params = params
        super().__init__(params, {"lr": lr, "betas": betas, "eps": eps, "weight_decay": weight_decay, "gradient_clipping": gradient_clipping, "max_gradient": max_gradient})


class PartialRowWiseLAMB(_Marker):
    def __init__(self, params, lr: float = 1e-2, betas: Tuple[float, float] = (0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0, gradient_clipping: bool = False, max_gradient: float = 1.0) -> None:
        self._params = params
        super().__init__(params, {"lr": lr, "betas": betas, "eps": eps, "weight_decay": weight_decay, "gradient_clipping": gradient_clipping, "max_gradient": max_gradient})


class Adam(_Marker):
    def __init__(self, params, lr: float = 1e-2, betas: Tuple[float, float] = (0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0, gradient_clipping: bool = False, max_gradient: float = 1.0) -> None:
        self._params = params
        super().__init__(params, {"lr": lr, "betas": betas, "eps": eps, "weight_decay": weight_decay, "gradient_clipping": gradient_clipping, "max_gradient": max_gradient})


class PartialRowWiseAdam(_Marker):
    def __init__(self, params, lr: float = 1e-2, betas: Tuple[float, float] = (0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0, gradient_clipping: bool = False, max_gradient: float = 1.0) -> None:
        self._params = params
        super().__init__(params, {"lr": lr, "betas": betas, "eps": eps, "weight_decay": weight_decay, "gradient_clipping": gradient_clipping, "max_gradient": max_gradient})


class Adagrad(_Marker):
    def __init__(self, params, lr: float = 1e-2, lr_decay: float = 0, weight_decay: float = 0, initial_accumulator_value: float = 0, eps: float = 1e-10, gradient_clipping: bool = False, max_gradient: float = 1.0) -> None:
        self._params = params
        super().__init__(params, {"lr": lr, "lr_decay": lr_decay, "weight_decay": weight_decay, "initial_accumulator_value": initial_accumulator_value, "eps": eps, "gradient_clipping": gradient_clipping, "max_gradient": max_gradient})
