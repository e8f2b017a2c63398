"""Learning-rate schedules as an optimizer wrapper: a list of stages, each with a policy, a length in steps and a value;
the wrapper multiplies every param group's base ``lr`` by the stage's factor before each step.  Its own step counter is
part of the state dict (``torchrec/optim/warmup.py:23-162``)."""
from __future__ import annotations

import logging
import math
from dataclasses import dataclass
from enum import Enum, unique
from typing import Any, List, Tuple

import torch

from torchrec_b200.optim.keyed import KeyedOptimizer, OptimizerWrapper

logger = logging.getLogger(__name__)


@unique
class WarmupPolicy(Enum):
    NONE = "none"
    LINEAR = "linear"
    CONSTANT = "constant"
    POLY = "poly"
    STEP = "step"
    INVSQRT = "inv_sqrt"  # inverse square root
    COSINE_ANNEALING_WARM_RESTARTS = "cosine_annealing_warm_restarts"


@dataclass
class WarmupStage:
    policy: WarmupPolicy = WarmupPolicy.LINEAR
    max_iters: int = 1
    value: float = 1.0
    lr_scale: float = 1.0
    decay_iters: int = -1  # poly: length of the decay (default max_iters); step: interval; cosine: T_0
    sgdr_period: int = 1


def _lr_stages(stages: List[WarmupStage]) -> List[WarmupStage]:
    last = WarmupStage(policy=WarmupPolicy.NONE, max_iters=1 << 63, value=1.0)
    if len(stages) == 0:
        return [last]
    start = 0
    for s in stages:
        assert s.max_iters > start, f"Max iter of the stage {s} must be greater than the previous max iter {start}"
        start = s.max_iters
        if s.decay_iters <= 0:
            s.decay_iters = s.max_iters
    return stages + [last]


def _get_multiplier(stage: WarmupStage, iter: int) -> float:
    m = 1.0
    if stage.policy == WarmupPolicy.LINEAR:
        m = stage.value + (1.0 - stage.value) * iter / stage.max_iters
    elif stage.policy == WarmupPolicy.CONSTANT:
        m = stage.value
    elif stage.policy == WarmupPolicy.POLY:
        m = math.pow(1 - iter / stage.decay_iters, stage.value)
    elif stage.policy == WarmupPolicy.STEP:
        m = math.pow(stage.value, iter // stage.decay_iters)
    elif stage.policy == WarmupPolicy.INVSQRT:
        m = 1.0 / math.sqrt(iter)
    elif stage.policy == WarmupPolicy.COSINE_ANNEALING_WARM_RESTARTS:
        t0 = stage.sgdr_period
        t_cur = iter % t0
        m = stage.value + (1.0 - stage.value) * 0.5 * (1 + math.cos(math.pi * t_cur / t0))
    return m * stage.lr_scale


class WarmupOptimizer(OptimizerWrapper):
    def __init__(self, optimizer: KeyedOptimizer, stages: List[WarmupStage], lr: float = 0.1, lr_param: str = "lr", param_name: str = "__warmup") -> None:
        super().__init__(optimizer)
        self._stages = _lr_stages(stages)
        self._lr_param = lr_param
        self._lr = lr
        self._warmup_param = torch.nn.Parameter()
        self.params[param_name] = self._warmup_param  # type: ignore[index]
        # the step counter lives in the optimizer state so that it is checkpointed with it
        self.state[self._warmup_param] = {"warmup": torch.tensor([0], dtype=torch.long)}  # type: ignore[index]
        self._set_lr(0, 0)

    def _set_lr(self, iter_: int, stage_id: int) -> None:
        lr = self._lr * _get_multiplier(self._stages[stage_id], iter_)
        for group in self.param_groups:
            group[self._lr_param] = lr  # type: ignore[index]

    def _get_warmup_state(self) -> Tuple[int, int]:
        iter_ = int(self.state[self._warmup_param]["warmup"][0].item())
        stage_id = 0
        for i, s in enumerate(self._stages):
            if iter_ >= s.max_iters and i + 1 < len(self._stages):
                stage_id = i + 1
        return iter_, stage_id

    def post_load_state_dict(self) -> None:
        iter_, stage_id = self._get_warmup_state()
        logger.info(f"Warmup Optimizer set to iteration {iter_}")
        self._set_lr(iter_, stage_id)

    def step(self, closure: Any = None) -> None:
        super().step(closure)
        self.state[self._warmup_param]["warmup"] += 1
        iter_, stage_id = self._get_warmup_state()
        self._set_lr(iter_, stage_id)
