"""Examples per second seen by a task (tower) after ``warmup_steps`` updates (``torchrec/metrics/tower_qps.py``).
States: examples and seconds; the slowest rank's time counts (max over ranks), examples add up."""
from __future__ import annotations

import time
from typing import Any, List, Optional

import torch

from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace, MetricPrefix
from torchrec_b200.metrics.rec_metric import MetricComputationReport, RecMetric, RecMetricComputation

WARMUP_STEPS = 100
NUM_EXAMPLES = "num_examples"
WARMUP_EXAMPLES = "warmup_examples"
TIME_LAPSE = "time_lapse"


def _compute_tower_qps(num_examples: torch.Tensor, time_lapse: torch.Tensor) -> torch.Tensor:
    return torch.where(time_lapse <= 0.0, torch.zeros_like(num_examples), num_examples / time_lapse.clamp(min=1e-12)).double()


def _max_reduction(state: torch.Tensor) -> torch.Tensor:
    return torch.max(state, dim=0).values


class TowerQPSMetricComputation(RecMetricComputation):
    def __init__(self, *args: Any, warmup_steps: int = WARMUP_STEPS, **kwargs: Any) -> None:
        self._warmup_steps = warmup_steps
        super().__init__(*args, **kwargs)
        self._add_state(NUM_EXAMPLES, torch.zeros(self._n_tasks, dtype=torch.long), add_window_state=True, dist_reduce_fx="sum", persistent=True)
        self._add_state(WARMUP_EXAMPLES, torch.zeros(self._n_tasks, dtype=torch.long), add_window_state=False, dist_reduce_fx="sum", persistent=True)
        self._add_state(TIME_LAPSE, torch.zeros(self._n_tasks, dtype=torch.double), add_window_state=True, dist_reduce_fx=_max_reduction, persistent=True)
        self._previous_ts = 0.0
        self._steps = 0

    def update(self, *, predictions: Optional[torch.Tensor], labels: torch.Tensor, weights: Optional[torch.Tensor], **kwargs: Any) -> None:
        self._steps += 1
        n = labels.shape[-1]
        if self._steps <= self._warmup_steps:
            self.warmup_examples += n
            if self._steps == self._warmup_steps:
                self._previous_ts = time.monotonic()
            return
        ts = time.monotonic()
        lapse = torch.full((self._n_tasks,), ts - self._previous_ts, dtype=torch.double, device=labels.device)
        ex = torch.full((self._n_tasks,), n, dtype=torch.long, device=labels.device)
        self._previous_ts = ts
        self.num_examples += ex
        self.time_lapse += lapse
        self._aggregate_window_state(NUM_EXAMPLES, ex, n)
        self._aggregate_window_state(TIME_LAPSE, lapse, n)

    def _compute(self) -> List[MetricComputationReport]:
        return [
            MetricComputationReport(name=MetricName.TOWER_QPS, metric_prefix=MetricPrefix.LIFETIME, value=_compute_tower_qps(self.num_examples.double(), self.time_lapse)),
            MetricComputationReport(name=MetricName.TOWER_QPS, metric_prefix=MetricPrefix.WINDOW,
                                    value=_compute_tower_qps(self.get_window_state(NUM_EXAMPLES).double(), self.get_window_state(TIME_LAPSE))),
            MetricComputationReport(name=MetricName.TOTAL_EXAMPLES, metric_prefix=MetricPrefix.DEFAULT, value=(self.num_examples + self.warmup_examples).detach()),
        ]


class TowerQPSMetric(RecMetric):
    _namespace = MetricNamespace.TOWER_QPS
    _computation_class = TowerQPSMetricComputation

    def __init__(self, world_size, my_rank, batch_size, tasks, warmup_steps: int = WARMUP_STEPS, **kwargs: Any) -> None:
        if warmup_steps < 0:
            raise ValueError(f"warmup_steps must be non-negative, got {warmup_steps}")
        super().__init__(world_size, my_rank, batch_size, tasks, warmup_steps=warmup_steps, **kwargs)
