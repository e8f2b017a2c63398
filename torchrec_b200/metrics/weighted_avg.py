"""Weighted average of the predictions (``torchrec/metrics/weighted_avg.py``)."""
from __future__ import annotations

from typing import Dict

import torch

from torchrec_b200.metrics._sum_states import SumStatesComputation, safe_div
from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace
from torchrec_b200.metrics.rec_metric import RecMetric


def get_mean(value_sum: torch.Tensor, num_samples: torch.Tensor) -> torch.Tensor:
    return safe_div(value_sum, num_samples)


class WeightedAvgMetricComputation(SumStatesComputation):
    STATES = ("weighted_sum", "weighted_num_samples")

    def _states(self, labels, predictions, weights, **kwargs):
        return {"weighted_sum": (predictions * weights).sum(dim=-1), "weighted_num_samples": weights.sum(dim=-1)}

    def _values(self, s):
        return [(MetricName.WEIGHTED_AVG, get_mean(s["weighted_sum"], s["weighted_num_samples"]))]


class WeightedAvgMetric(RecMetric):
    _namespace = MetricNamespace.WEIGHTED_AVG
    _computation_class = WeightedAvgMetricComputation
