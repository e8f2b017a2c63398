"""Binary accuracy at a threshold (``torchrec/metrics/accuracy.py``)."""
from __future__ import annotations

from typing import Any, Dict

import torch

from torchrec_b200.metrics._sum_states import SumStatesComputation, safe_div
from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace
from torchrec_b200.metrics.rec_metric import RecMetric

THRESHOLD = "threshold"


def compute_accuracy(accuracy_sum: torch.Tensor, weighted_num_samples: torch.Tensor) -> torch.Tensor:
    return safe_div(accuracy_sum, weighted_num_samples)


def compute_accuracy_sum(labels: torch.Tensor, predictions: torch.Tensor, weights: torch.Tensor, threshold: float = 0.5) -> torch.Tensor:
    return (weights * ((predictions.double() >= threshold) == (labels >= 0.5)).double()).sum(dim=-1)


def get_accuracy_states(labels: torch.Tensor, predictions: torch.Tensor, weights: torch.Tensor, threshold: float = 0.5) -> Dict[str, torch.Tensor]:
    return {"accuracy_sum": compute_accuracy_sum(labels, predictions, weights, threshold), "weighted_num_samples": weights.sum(dim=-1)}


class AccuracyMetricComputation(SumStatesComputation):
    STATES = ("accuracy_sum", "weighted_num_samples")

    def __init__(self, *args: Any, threshold: float = 0.5, **kwargs: Any) -> None:
        self._threshold = threshold
        super().__init__(*args, **kwargs)

    def _states(self, labels, predictions, weights, **kwargs):
        return get_accuracy_states(labels, predictions, weights, self._threshold)

    def _values(self, s):
        return [(MetricName.ACCURACY, compute_accuracy(s["accuracy_sum"], s["weighted_num_samples"]))]


class AccuracyMetric(RecMetric):
    _namespace = MetricNamespace.ACCURACY
    _computation_class = AccuracyMetricComputation
