"""Calibration-free NE: NE divided by the entropy term evaluated at the mean prediction, which removes the
effect of a global mis-calibration (``torchrec/metrics/cali_free_ne.py:65-89``)."""
from __future__ import annotations

from typing import Any, Dict

import torch

from torchrec_b200.metrics._sum_states import SumStatesComputation
from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace
from torchrec_b200.metrics.ne import compute_ne, get_ne_states
from torchrec_b200.metrics.rec_metric import RecMetric


def compute_cali_free_ne(ce_sum, weighted_num_samples, pos_labels, neg_labels, weighted_sum_predictions, eta, allow_missing_label_with_zero_weight=False):
    if allow_missing_label_with_zero_weight and not bool(weighted_num_samples.all()):
        return torch.full_like(ce_sum, eta)
    raw = compute_ne(ce_sum, weighted_num_samples, pos_labels, neg_labels, eta)
    mean_pred = weighted_sum_predictions / weighted_num_samples
    return raw / (-pos_labels * torch.log2(mean_pred) - (weighted_num_samples - pos_labels) * torch.log2(1 - mean_pred))


def get_cali_free_ne_states(labels: torch.Tensor, predictions: torch.Tensor, weights: torch.Tensor, eta: float) -> Dict[str, torch.Tensor]:
    """The NE states plus the weighted sum of predictions (the mean prediction is what the calibration-free form divides out)."""
    states = get_ne_states(labels, predictions, weights, eta)
    states["weighted_sum_predictions"] = (weights * predictions).sum(dim=-1)
    return states


class CaliFreeNEMetricComputation(SumStatesComputation):
    STATES = ("cross_entropy_sum", "weighted_num_samples", "pos_labels", "neg_labels", "weighted_sum_predictions")

    def __init__(self, *args: Any, allow_missing_label_with_zero_weight: bool = False, **kwargs: Any) -> None:
        self._allow_missing = allow_missing_label_with_zero_weight
        super().__init__(*args, **kwargs)
        self.eta = 1e-12

    def _states(self, labels, predictions, weights, **kwargs):
        return get_cali_free_ne_states(labels, predictions, weights, self.eta)

    def _values(self, s):
        return [(MetricName.CALI_FREE_NE, compute_cali_free_ne(
            s["cross_entropy_sum"], s["weighted_num_samples"], s["pos_labels"], s["neg_labels"], s["weighted_sum_predictions"], self.eta, self._allow_missing))]


class CaliFreeNEMetric(RecMetric):
    _namespace = MetricNamespace.CALI_FREE_NE
    _computation_class = CaliFreeNEMetricComputation
