"""Binary precision at a threshold (``torchrec/metrics/precision.py``)."""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch

from torchrec_b200.metrics._sum_states import SumStatesComputation, safe_div
from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace
from torchrec_b200.metrics.rec_metric import RecMetric


def compute_precision(num_true_positives: torch.Tensor, num_false_positives: torch.Tensor) -> torch.Tensor:
    return safe_div(num_true_positives, num_true_positives + num_false_positives)


def compute_true_pos_sum(labels: torch.Tensor, predictions: torch.Tensor, weights: torch.Tensor, threshold: float = 0.5) -> torch.Tensor:
    """Weight of the positives predicted at or above the threshold, per task."""
    return (weights * (predictions.double() >= threshold) * labels).sum(dim=-1)


def compute_false_pos_sum(labels: torch.Tensor, predictions: torch.Tensor, weights: torch.Tensor, threshold: float = 0.5) -> torch.Tensor:
    """Weight of the negatives predicted at or above the threshold, per task."""
    return (weights * (predictions.double() >= threshold) * (1 - labels)).sum(dim=-1)


def get_precision_states(labels: torch.Tensor, predictions: torch.Tensor, weights: Optional[torch.Tensor], threshold: float = 0.5) -> Dict[str, torch.Tensor]:
    if weights is None:
        weights = torch.ones_like(predictions)
    return {"true_pos_sum": compute_true_pos_sum(labels, predictions, weights, threshold),
            "false_pos_sum": compute_false_pos_sum(labels, predictions, weights, threshold)}


class PrecisionMetricComputation(SumStatesComputation):
    STATES = ("true_pos_sum", "false_pos_sum")

    def __init__(self, *args: Any, threshold: float = 0.5, **kwargs: Any) -> None:
        self._threshold = threshold
        super().__init__(*args, **kwargs)

    def _states(self, labels, predictions, weights, **kwargs):
        return get_precision_states(labels, predictions, weights, self._threshold)

    def _values(self, s):
        return [(MetricName.PRECISION, compute_precision(s["true_pos_sum"], s["false_pos_sum"]))]


class PrecisionMetric(RecMetric):
    _namespace = MetricNamespace.PRECISION
    _computation_class = PrecisionMetricComputation
