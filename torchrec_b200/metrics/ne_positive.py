"""Normalized entropy restricted to the positive examples' cross entropy (``torchrec/metrics/ne_positive.py``)."""
from __future__ import annotations

from typing import Any, Dict

import torch

from torchrec_b200.metrics._sum_states import SumStatesComputation
from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace
from torchrec_b200.metrics.ne import base_rate_entropy
from torchrec_b200.metrics.rec_metric import RecMetric


def compute_cross_entropy_positive(labels, predictions, weights, eta):
    p = predictions.double().clamp(min=eta, max=1 - eta)
    return -weights * labels * torch.log2(p)


def compute_ne_positive(ce_positive_sum: torch.Tensor, weighted_num_samples: torch.Tensor, pos_labels: torch.Tensor, neg_labels: torch.Tensor,
                        eta: float, allow_missing_label_with_zero_weight: bool = False) -> torch.Tensor:
    """Cross entropy of the positives over the entropy of the base rate; ``eta`` for every task when a task has no weight and
    missing labels are allowed (``torchrec/metrics/ne_positive.py:48-65``)."""
    if allow_missing_label_with_zero_weight and not bool(weighted_num_samples.all()):
        return torch.full_like(weighted_num_samples, eta)
    return ce_positive_sum / base_rate_entropy(pos_labels, neg_labels, weighted_num_samples, eta)


def get_ne_positive_states(labels: torch.Tensor, predictions: torch.Tensor, weights: torch.Tensor, eta: float) -> Dict[str, torch.Tensor]:
    return {
        "cross_entropy_positive_sum": compute_cross_entropy_positive(labels, predictions, weights, eta).sum(dim=-1),
        "weighted_num_samples": weights.sum(dim=-1),
        "pos_labels": (weights * labels).sum(dim=-1),
        "neg_labels": (weights * (1.0 - labels)).sum(dim=-1),
    }


class NEPositiveMetricComputation(SumStatesComputation):
    STATES = ("cross_entropy_positive_sum", "weighted_num_samples", "pos_labels", "neg_labels")

    def __init__(self, *args: Any, allow_missing_label_with_zero_weight: bool = False, **kwargs: Any) -> None:
        self._allow_missing = allow_missing_label_with_zero_weight
        super().__init__(*args, **kwargs)
        self.eta = 1e-12

    def _states(self, labels, predictions, weights, **kwargs):
        return get_ne_positive_states(labels, predictions, weights, self.eta)

    def _values(self, s):
        return [(MetricName.NE_POSITIVE, compute_ne_positive(s["cross_entropy_positive_sum"], s["weighted_num_samples"], s["pos_labels"],
                                                             s["neg_labels"], self.eta, self._allow_missing))]


class NEPositiveMetric(RecMetric):
    _namespace = MetricNamespace.NE_POSITIVE
    _computation_class = NEPositiveMetricComputation
