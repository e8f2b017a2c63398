"""Binary recall at a threshold (``torchrec/metrics/recall.py``)."""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch

from torchrec_b200.metrics._sum_states import SumStatesComputation, safe_div
from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace
from torchrec_b200.metrics.rec_metric import RecMetric


def compute_recall(num_true_positives: torch.Tensor, num_false_negitives: torch.Tensor) -> torch.Tensor:
    return safe_div(num_true_positives, num_true_positives + num_false_negitives)


def compute_true_pos_sum(labels: torch.Tensor, predictions: torch.Tensor, weights: torch.Tensor, threshold: float = 0.5) -> torch.Tensor:
    """Weight of the positives predicted at or above the threshold, per task."""
    return (weights * (predictions.double() >= threshold) * labels).sum(dim=-1)


def compute_false_neg_sum(labels: torch.Tensor, predictions: torch.Tensor, weights: torch.Tensor, threshold: float = 0.5) -> torch.Tensor:
    """Weight of the positives predicted at or below the threshold, per task (a prediction equal to the threshold counts on both
    sides, as in ``torchrec/metrics/recall.py:45-52``)."""
    return (weights * (predictions.double() <= threshold) * labels).sum(dim=-1)


def get_recall_states(labels: torch.Tensor, predictions: torch.Tensor, weights: Optional[torch.Tensor], threshold: float = 0.5) -> Dict[str, torch.Tensor]:
    if weights is None:
        weights = torch.ones_like(predictions)
    return {"true_pos_sum": compute_true_pos_sum(labels, predictions, weights, threshold),
            "false_neg_sum": compute_false_neg_sum(labels, predictions, weights, threshold)}


class RecallMetricComputation(SumStatesComputation):
    STATES = ("true_pos_sum", "false_neg_sum")

    def __init__(self, *args: Any, threshold: float = 0.5, **kwargs: Any) -> None:
        self._threshold = threshold
        super().__init__(*args, **kwargs)

    def _states(self, labels, predictions, weights, **kwargs):
        return get_recall_states(labels, predictions, weights, self._threshold)

    def _values(self, s):
        return [(MetricName.RECALL, compute_recall(s["true_pos_sum"], s["false_neg_sum"]))]


class RecallMetric(RecMetric):
    _namespace = MetricNamespace.RECALL
    _computation_class = RecallMetricComputation
