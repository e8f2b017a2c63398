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
    """Validated stage list with an open-ended identity stage appended (what applies after the last boundary)."""
    boundary = 0
    for stage in stages:
        assert stage.max_iters > boundary, f"Max iter of the stage {stage} must be greater than the previous max iter {boundary}"
        boundary = stage.max_iters
        if stage.decay_iters <= 0:
            stage.decay_iters = stage.max_iters
    return list(stages) + [WarmupStage(policy=WarmupPolicy.NONE, max_iters=1 << 63, value=1.0)]


def _cosine_restart(stage: WarmupStage, it: int) -> float:
    phase = (it % stage.sgdr_period) / stage.sgdr_period
    return stage.value + (1.0 - stage.value) * 0.5 * (1.0 + math.cos(math.pi * phase))


_FACTOR = {
    WarmupPolicy.NONE: lambda s, it: 1.0,
    WarmupPolicy.LINEAR: lambda s, it: s.value + (1.0 - s.value) * it / s.max_iters,
    WarmupPolicy.CONSTANT: lambda s, it: s.value,
    WarmupPolicy.POLY: lambda s, it: (1.0 - it / s.decay_iters) ** s.value,
    WarmupPolicy.STEP: lambda s, it: s.value ** (it // s.decay_iters),
    WarmupPolicy.INVSQRT: lambda s, it: 1.0 / math.sqrt(it),
    WarmupPolicy.COSINE_ANNEALING_WARM_RESTARTS: _cosine_restart,
}


def _get_multiplier(stage: WarmupStage, iter: int) -> float:
    return _FACTOR[stage.policy](stage, iter) * stage.lr_scale


class WarmupOptimizer(OptimizerWrapper):
    def __init__(self, optimizer: KeyedOptimizer, stages: List[WarmupStage], lr: float = 0.1, lr_param: str = "lr", param_name: str = "__warmup") -> None:
        super().__init__(optimizer)
        self._stages = _lr_stages(stages)
        self._lr_param, self._lr = lr_param, lr
        # the step counter is the state of a dummy parameter, so it is checkpointed with the optimizer
        self._warmup_param = torch.nn.Parameter()
        self.params[param_name] = self._warmup_param  # type: ignore[index]
        self.state[self._warmup_param] = {"warmup": torch.zeros(1, dtype=torch.long)}  # type: ignore[index]
        self._apply(0)

    def _counter(self) -> torch.Tensor:
        return self.state[self._warmup_param]["warmup"]

    def _stage_of(self, it: int) -> WarmupStage:
        for stage in self._stages:
            if it < stage.max_iters:
                return stage
        return self._stages[-1]

    def _apply(self, it: int) -> None:
        value = self._lr * _get_multiplier(self._stage_of(it), it)
        for group in self.param_groups:
            group[self._lr_param] = value  # type: ignore[index]

    def _get_warmup_state(self) -> Tuple[int, int]:
        it = int(self._counter()[0])
        return it, self._stages.index(self._stage_of(it))

    def post_load_state_dict(self) -> None:
        it = int(self._counter()[0])
        logger.info(f"Warmup Optimizer set to iteration {it}")
        self._apply(it)

    def step(self, closure: Any = None) -> None:
        super().step(closure)
        self._counter().add_(1)
        self._apply(int(self._counter()[0]))
