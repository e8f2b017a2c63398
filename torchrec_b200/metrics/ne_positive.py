"""Normalized entropy restricted to the positive examples' cross entropy (``torchrec/metrics/ne_positive.py``)."""
from __future__ import annotations

from typing import Any

import torch

from torchrec_b200.metrics._sum_states import SumStatesComputation
from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace
from torchrec_b200.metrics.ne import base_rate_entropy
from torchrec_b200.metrics.rec_metric import RecMetric


def compute_cross_entropy_positive(labels, predictions, weights, eta):
    p = predictions.double().clamp(min=eta, max=1 - eta)
    return -weights * labels * torch.log2(p)


class NEPositiveMetricComputation(SumStatesComputation):
    STATES = ("cross_entropy_positive_sum", "weighted_num_samples", "pos_labels", "neg_labels")

    def __init__(self, *args: Any, allow_missing_label_with_zero_weight: bool = False, **kwargs: Any) -> None:
        self._allow_missing = allow_missing_label_with_zero_weight
        super().__init__(*args, **kwargs)
        self.eta = 1e-12

    def _states(self, labels, predictions, weights, **kwargs):
        return {
            "cross_entropy_positive_sum": compute_cross_entropy_positive(labels, predictions, weights, self.eta).sum(dim=-1),
            "weighted_num_samples": weights.sum(dim=-1),
            "pos_labels": (weights * labels).sum(dim=-1),
            "neg_labels": (weights * (1.0 - labels)).sum(dim=-1),
        }

    def _values(self, s):
        if self._allow_missing and not bool(s["weighted_num_samples"].all()):
            v = torch.full_like(s["weighted_num_samples"], self.eta)
        else:
            v = s["cross_entropy_positive_sum"] / base_rate_entropy(s["pos_labels"], s["neg_labels"], s["weighted_num_samples"], self.eta)
        return [(MetricName.NE_POSITIVE, v)]


class NEPositiveMetric(RecMetric):
    _namespace = MetricNamespace.NE_POSITIVE
    _computation_class = NEPositiveMetricComputation
