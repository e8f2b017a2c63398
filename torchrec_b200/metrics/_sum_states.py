"""Shared base for metrics whose states are plain sums over examples (NE, calibration, CTR, MSE, ...).

A subclass lists its state names, computes the per-update contribution of every state from
``(labels, predictions, weights)`` and maps a ``{state: tensor}`` dict to reported values; the lifetime and
window bookkeeping is identical for all of them and lives here.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch

from torchrec_b200.metrics.metrics_namespace import MetricNameBase, MetricPrefix
from torchrec_b200.metrics.rec_metric import MetricComputationReport, RecMetricComputation, RecMetricException


class SumStatesComputation(RecMetricComputation):
    STATES: Tuple[str, ...] = ()
    NEEDS_PREDICTIONS: bool = True

    def __init__(self, *args: Any, **kwargs: Any) -> None:
        super().__init__(*args, **kwargs)
        for s in self.STATES:
            self._add_state(s, torch.zeros(self._state_shape(s), dtype=torch.double), add_window_state=True, dist_reduce_fx="sum", persistent=True)

    def _state_shape(self, name: str) -> Tuple[int, ...]:
        return (self._n_tasks,)

    # -- to implement --------------------------------------------------------------------------------
    def _states(self, labels: torch.Tensor, predictions: Optional[torch.Tensor], weights: torch.Tensor, **kwargs: Any) -> Dict[str, torch.Tensor]:
        raise NotImplementedError

    def _values(self, s: Dict[str, torch.Tensor]) -> List[Tuple[MetricNameBase, torch.Tensor]]:
        raise NotImplementedError

    # -- shared --------------------------------------------------------------------------------------
    def update(self, *, predictions: Optional[torch.Tensor], labels: torch.Tensor, weights: Optional[torch.Tensor], **kwargs: Any) -> None:
        if self.NEEDS_PREDICTIONS and predictions is None:
            raise RecMetricException(f"Inputs 'predictions' should not be None for {type(self).__name__} update")
        if weights is None:
            weights = torch.ones_like(labels, dtype=torch.float32)
        n = labels.shape[-1]
        # states are double sums: promote the per-example inputs once so that no partial sum is taken in float32
        weights = weights.double()
        labels = labels.double()
        for name, value in self._states(labels, predictions, weights, **kwargs).items():
            state = getattr(self, name)
            value = value.to(state.dtype)
            state += value
            self._aggregate_window_state(name, value, n)

    def _compute(self) -> List[MetricComputationReport]:
        life = {s: getattr(self, s) for s in self.STATES}
        win = {s: self.get_window_state(s) for s in self.STATES}
        reports: List[MetricComputationReport] = []
        for prefix, states in ((MetricPrefix.LIFETIME, life), (MetricPrefix.WINDOW, win)):
            for name, value in self._values(states):
                reports.append(MetricComputationReport(name=name, metric_prefix=prefix, value=value))
        return reports


def safe_div(num: torch.Tensor, den: torch.Tensor, default: float = 0.0) -> torch.Tensor:
    return torch.where(den == 0, torch.full_like(num, default, dtype=torch.double), num.double() / den.double().clamp(min=torch.finfo(torch.double).tiny))
