"""Hindsight target precision/recall: the lowest of 1000 thresholds whose precision reaches ``target_precision``, and the
precision / recall there (``torchrec/metrics/hindsight_target_pr.py``).  Single-task computation."""
from __future__ import annotations

from typing import Any, List, Optional, Tuple

import torch

from torchrec_b200.metrics._sum_states import SumStatesComputation, safe_div
from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace, MetricPrefix
from torchrec_b200.metrics.rec_metric import MetricComputationReport, RecMetric

THRESHOLD_GRANULARITY = 1000
TARGET_PRECISION = "target_precision"


def compute_threshold_idx(num_true_positives: torch.Tensor, num_false_positives: torch.Tensor, target_precision: float) -> int:
    precision = safe_div(num_true_positives, num_true_positives + num_false_positives)
    ok = torch.nonzero(precision >= target_precision)
    return int(ok[0]) if ok.numel() else THRESHOLD_GRANULARITY - 1


def _sum_over_thresholds(predictions: torch.Tensor, mass: torch.Tensor, above: bool) -> torch.Tensor:
    """``out[i] = sum(mass[predictions >= t_i])`` (or ``<=``) for the 1000 thresholds, as one [thresholds, samples] comparison."""
    p = predictions.double().view(-1)
    thr = torch.linspace(0, 1, steps=THRESHOLD_GRANULARITY, dtype=torch.double, device=p.device).unsqueeze(1)
    side = (p.unsqueeze(0) >= thr) if above else (p.unsqueeze(0) <= thr)
    return (side * mass.double().view(1, -1)).sum(-1)


def compute_true_pos_sum(labels: torch.Tensor, predictions: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    return _sum_over_thresholds(predictions, weights * labels, above=True)


def compute_false_pos_sum(labels: torch.Tensor, predictions: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    return _sum_over_thresholds(predictions, weights * (1 - labels), above=True)


def compute_false_neg_sum(labels: torch.Tensor, predictions: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    return _sum_over_thresholds(predictions, weights * labels, above=False)


def get_pr_states(labels: torch.Tensor, predictions: torch.Tensor, weights: Optional[torch.Tensor]):
    if weights is None:
        weights = torch.ones_like(predictions)
    return {"true_pos_sum": compute_true_pos_sum(labels, predictions, weights), "false_pos_sum": compute_false_pos_sum(labels, predictions, weights),
            "false_neg_sum": compute_false_neg_sum(labels, predictions, weights)}


class HindsightTargetPRMetricComputation(SumStatesComputation):
    STATES = ("true_pos_sum", "false_pos_sum", "false_neg_sum")

    def __init__(self, *args: Any, target_precision: float = 0.5, **kwargs: Any) -> None:
        self._target_precision = target_precision
        super().__init__(*args, **kwargs)

    def _state_shape(self, name: str) -> Tuple[int, ...]:
        return (THRESHOLD_GRANULARITY,)

    def _states(self, labels, predictions, weights, **kwargs):
        return get_pr_states(labels, predictions, weights)

    def _compute(self) -> List[MetricComputationReport]:
        reports = []
        for prefix, get in ((MetricPrefix.LIFETIME, lambda n: getattr(self, n)), (MetricPrefix.WINDOW, self.get_window_state)):
            tp, fp, fn = get("true_pos_sum"), get("false_pos_sum"), get("false_neg_sum")
            i = compute_threshold_idx(tp, fp, self._target_precision)
            reports += [
                MetricComputationReport(name=MetricName.HINDSIGHT_TARGET_PR, metric_prefix=prefix, value=torch.tensor([float(i)], dtype=torch.double)),
                MetricComputationReport(name=MetricName.HINDSIGHT_TARGET_PRECISION, metric_prefix=prefix, value=safe_div(tp[i], tp[i] + fp[i]).view(1)),
                MetricComputationReport(name=MetricName.HINDSIGHT_TARGET_RECALL, metric_prefix=prefix, value=safe_div(tp[i], tp[i] + fn[i]).view(1)),
            ]
        return reports


class HindsightTargetPRMetric(RecMetric):
    _namespace = MetricNamespace.HINDSIGHT_TARGET_PR
    _computation_class = HindsightTargetPRMetricComputation
