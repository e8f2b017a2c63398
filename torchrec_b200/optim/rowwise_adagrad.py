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


class RowWiseAdagrad(Optimizer):
    def __init__(self, params: Iterable[torch.nn.Parameter], lr: float = 1e-2, lr_decay: float = 0.0, weight_decay: float = 0.0,
                 initial_accumulator_value: float = 0.0, eps: float = 1e-10, *, maximize: bool = False, **unused) -> None:
        if not 0.0 <= lr:
            raise ValueError(f"Invalid learning rate: {lr}")
        if not 0.0 <= lr_decay:
            raise ValueError(f"Invalid lr_decay value: {lr_decay}")
        if not 0.0 <= weight_decay:
            raise ValueError(f"Invalid weight_decay value: {weight_decay}")
        if not 0.0 <= initial_accumulator_value:
            raise ValueError(f"Invalid initial_accumulator_value value: {initial_accumulator_value}")
        if not 0.0 <= eps:
            raise ValueError(f"Invalid epsilon value: {eps}")
        defaults = dict(lr=lr, lr_decay=lr_decay, eps=eps, weight_decay=weight_decay, initial_accumulator_value=initial_accumulator_value, maximize=maximize)
        super().__init__(params, defaults)
        for group in self.param_groups:
            for p in group["params"]:
                state = self.state[p]
                state["step"] = torch.tensor(0.0)
                init_value = complex(initial_accumulator_value, initial_accumulator_value) if torch.is_complex(p) else initial_accumulator_value
                state["sum"] = (
                    torch.full_like(p, init_value, memory_format=torch.preserve_format).mean(axis=1).view(-1, 1)
                    if p.dim() > 1 else torch.full_like(p, init_value, memory_format=torch.preserve_format)
                )

    def __setstate__(self, state: Dict[str, Any]) -> None:
        super().__setstate__(state)
        for group in self.param_groups:
            group.setdefault("maximize", False)
        state_values = list(self.state.values())
        if state_values and not torch.is_tensor(state_values[0]["step"]):
            for s in state_values:
                s["step"] = torch.tensor(float(s["step"]))

    def share_memory(self) -> None:
        for group in self.param_groups:
            for p in group["params"]:
                self.state[p]["sum"].share_memory_()

    @torch.no_grad()
    def step(self, closure: Any = None) -> Any:
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            params_with_grad, grads, state_sums, state_steps = [], [], [], []
            for p in group["params"]:
                if p.grad is not None:
                    params_with_grad.append(p)
                    grads.append(p.grad)
                    state = self.state[p]
                    state_sums.append(state["sum"])
                    state_steps.append(state["step"])
            adagrad(params_with_grad, grads, state_sums, state_steps, lr=group["lr"], weight_decay=group["weight_decay"],
                    lr_decay=group["lr_decay"], eps=group["eps"], maximize=group["maximize"])
        return loss


def adagrad(params: List[Tensor], grads: List[Tensor], state_sums: List[Tensor], state_steps: List[Tensor], *, lr: float,
            weight_decay: float, lr_decay: float, eps: float, maximize: bool) -> None:
    for param, grad, state_sum, step_t in zip(params, grads, state_sums, state_steps):
        if grad.is_sparse:
            raise RuntimeError("RowWise adagrad cannot be used with sparse gradients")
        step_t += 1
        step = step_t.item()
        grad = grad if not maximize else -grad
        if weight_decay != 0:
            grad = grad.add(param, alpha=weight_decay)
        state_sum += grad.pow(2).mean(axis=1).view(-1, 1)
        std = state_sum.sqrt().add_(eps)
        clr = lr / (1 + (step - 1) * lr_decay)
        param.addcdiv_(grad, std, value=-clr)
