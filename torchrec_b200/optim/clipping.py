"""Gradient clipping as an optimizer wrapper: clip, then step the wrapped optimizer.

NORM clipping computes ONE global norm over all parameters: replicated parameters contribute their local norm once,
sharded parameters (tables split over ranks) contribute the sum of the shard norms over the process group
(an all-reduce of the p-th power sums).  Counterpart of ``torchrec/optim/clipping.py`` (``GradientClippingOptimizer``,
sharded norm ``:243-272``).
"""
from __future__ import annotations

from enum import Enum, unique
from typing import Any, Dict, List, Optional, Union

import torch
import torch.distributed as dist

from torchrec_b200.optim.keyed import KeyedOptimizer, OptimizerWrapper


@unique
class GradientClipping(Enum):
    NORM = "norm"
    VALUE = "value"
    NONE = "none"


def _total_norm(grads: List[torch.Tensor], norm_type: float, pg: Optional[dist.ProcessGroup], sharded: bool) -> torch.Tensor:
    if not grads:
        return torch.tensor(0.0)
    if norm_type == float("inf"):
        total = torch.stack([g.detach().abs().max() for g in grads]).max()
        if sharded and dist.is_available() and dist.is_initialized():
            dist.all_reduce(total, op=dist.ReduceOp.MAX, group=pg)
        return total
    total = torch.stack([torch.linalg.vector_norm(g.detach().float(), norm_type) ** norm_type for g in grads]).sum()
    if sharded and dist.is_available() and dist.is_initialized():
        dist.all_reduce(total, op=dist.ReduceOp.SUM, group=pg)
    return total


class GradientClippingOptimizer(OptimizerWrapper):
    """``clipping``: NORM (scale all gradients so the global ``norm_type`` norm is at most ``max_gradient``), VALUE (clamp
    every element to ``[-max_gradient, max_gradient]``) or NONE."""

    def __init__(self, optimizer: KeyedOptimizer, clipping: GradientClipping = GradientClipping.NONE, max_gradient: float = 0.1,
                 norm_type: Union[float, str] = 2.0, enable_global_grad_clip: bool = False, param_to_pgs: Optional[Dict[torch.nn.Parameter, List[dist.ProcessGroup]]] = None) -> None:
        super().__init__(optimizer)
        self._clipping = clipping
        self._max_gradient = max_gradient
        self._norm_type = float(norm_type)
        self._check_meta = True
        self._enable_global_grad_clip = enable_global_grad_clip
        self._step_num = 0
        self._params: List[torch.Tensor] = []
        self._replicate_params: List[torch.Tensor] = []
        self._sharded_params: List[torch.Tensor] = []
        for group in self.param_groups:
            for p in group["params"]:
                self._params.append(p)
                # parameters that only exist as this rank's shard of a larger tensor
                if getattr(p, "_is_sharded", False) or type(p).__name__ in ("ShardedTensor", "DTensor"):
                    self._sharded_params.append(p)
                else:
                    self._replicate_params.append(p)
        self._last_total_norm: Optional[torch.Tensor] = None

    def step(self, closure: Any = None) -> None:
        self._step_num += 1
        if self._check_meta:
            if any(getattr(p, "is_meta", False) for p in self._params):
                self._check_meta = False
                super().step(closure)
                return
            self._check_meta = False
        if self._clipping == GradientClipping.NORM:
            self._clip_norm()
        elif self._clipping == GradientClipping.VALUE:
            torch.nn.utils.clip_grad_value_([p for p in self._params if p.grad is not None], clip_value=self._max_gradient)
        super().step(closure)

    def _clip_norm(self) -> None:
        rep = [p.grad for p in self._replicate_params if p.grad is not None]
        shd = [p.grad for p in self._sharded_params if p.grad is not None]
        if not rep and not shd:
            return
        if not self._enable_global_grad_clip and not shd:
            self._last_total_norm = torch.nn.utils.clip_grad_norm_([p for p in self._replicate_params if p.grad is not None], self._max_gradient, norm_type=self._norm_type)
            return
        dev = (rep + shd)[0].device
        r = _total_norm(rep, self._norm_type, None, False).to(dev)
        s = _total_norm(shd, self._norm_type, None, True).to(dev)
        total = torch.maximum(r, s) if self._norm_type == float("inf") else (r + s) ** (1.0 / self._norm_type)
        self._last_total_norm = total
        coef = torch.clamp(self._max_gradient / (total + 1e-6), max=1.0)
        for g in rep + shd:
            g.detach().mul_(coef.to(g.device))
