"""Row-wise Adagrad as a plain torch optimizer: one accumulator per embedding row.

``sum_r += mean(g_r^2)``; ``w_r -= lr * g_r / (sqrt(sum_r) + eps)``.  It is the python statement
of the update the TBE kernel fuses (cf. ``torchrec/optim/rowwise_adagrad.py:23-232``) and serves as
its oracle.  Note the dense form updates every row each step; the fused kernel only touches rows
that received a gradient, which differs when ``weight_decay != 0``.
"""
from __future__ import annotations

import logging
from typing import Any, Dict, Iterable, List

import torch
from torch import Tensor
from torch.optim.optimizer import Optimizer

logger: logging.Logger = logging.getLogger(__name__)

_NON_NEGATIVE = (("lr", "learning rate"), ("lr_decay", "lr_decay value"), ("weight_decay", "weight_decay value"),
                 ("initial_accumulator_value", "initial_accumulator_value value"), ("eps", "epsilon value"))


def _row_state(p: Tensor, fill: float) -> Tensor:
    """One accumulator per row of a matrix (kept as a column so that it broadcasts), one per element otherwise."""
    if p.dim() > 1:
        return torch.full((p.shape[0], 1), fill, dtype=p.dtype, device=p.device)
    return torch.full_like(p, fill, memory_format=torch.preserve_format)


def _update_one(param: Tensor, grad: Tensor, acc: Tensor, steps: Tensor, lr: float, weight_decay: float, lr_decay: float, eps: float, maximize: bool) -> None:
    if grad.is_sparse:
        raise RuntimeError("RowWise adagrad cannot be used with sparse gradients")
    steps += 1
    g = grad.neg() if maximize else grad
    if weight_decay != 0:
        g = g + weight_decay * param
    acc.add_(g.square().mean(dim=1, keepdim=True))
    rate = lr / (1.0 + (float(steps) - 1.0) * lr_decay)
    param.addcdiv_(g, acc.sqrt() + eps, value=-rate)


class RowWiseAdagrad(Optimizer):
    def __init__(self, params: Iterable[torch.nn.Parameter], lr: float = 1e-2, lr_decay: float = 0.0, weight_decay: float = 0.0,
                 initial_accumulator_value: float = 0.0, eps: float = 1e-10, *, maximize: bool = False, **unused) -> None:
        given = dict(lr=lr, lr_decay=lr_decay, weight_decay=weight_decay, initial_accumulator_value=initial_accumulator_value, eps=eps)
        for key, label in _NON_NEGATIVE:
            if given[key] < 0.0:
                raise ValueError(f"Invalid {label}: {given[key]}")
        super().__init__(params, dict(given, maximize=maximize))
        for p in self._all_params():
            fill = complex(initial_accumulator_value, initial_accumulator_value) if torch.is_complex(p) else initial_accumulator_value
            self.state[p].update(step=torch.tensor(0.0), sum=_row_state(p, fill))

    def _all_params(self) -> Iterable[Tensor]:
        for group in self.param_groups:
            yield from group["params"]

    def __setstate__(self, state: Dict[str, Any]) -> None:
        super().__setstate__(state)
        for group in self.param_groups:
            group.setdefault("maximize", False)
        for entry in self.state.values():  # checkpoints written with a python number as step counter
            if not torch.is_tensor(entry["step"]):
                entry["step"] = torch.tensor(float(entry["step"]))

    def share_memory(self) -> None:
        for p in self._all_params():
            self.state[p]["sum"].share_memory_()

    @torch.no_grad()
    def step(self, closure: Any = None) -> Any:
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            live = [p for p in group["params"] if p.grad is not None]
            adagrad(live, [p.grad for p in live], [self.state[p]["sum"] for p in live], [self.state[p]["step"] for p in live],
                    lr=group["lr"], weight_decay=group["weight_decay"], lr_decay=group["lr_decay"], eps=group["eps"], maximize=group["maximize"])
        return loss


def adagrad(params: List[Tensor], grads: List[Tensor], state_sums: List[Tensor], state_steps: List[Tensor], *, lr: float,
            weight_decay: float, lr_decay: float, eps: float, maximize: bool) -> None:
    """Functional form over parallel lists (the signature of ``torchrec.optim.rowwise_adagrad.adagrad``)."""
    for quad in zip(params, grads, state_sums, state_steps):
        _update_one(*quad, lr, weight_decay, lr_decay, eps, maximize)
