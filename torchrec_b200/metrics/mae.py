"""Mean absolute error (``torchrec/metrics/mae.py``)."""
from __future__ import annotations

from typing import Dict

import torch

from torchrec_b200.metrics._sum_states import SumStatesComputation, safe_div
from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace
from torchrec_b200.metrics.rec_metric import RecMetric

ERROR_SUM = "error_sum"
WEIGHTED_NUM_SAMPES = "weighted_num_samples"


def compute_mae(error_sum: torch.Tensor, weighted_num_samples: torch.Tensor) -> torch.Tensor:
    return safe_div(error_sum, weighted_num_samples)


def get_mae_states(labels: torch.Tensor, predictions: torch.Tensor, weights: torch.Tensor) -> Dict[str, torch.Tensor]:
    return {ERROR_SUM: (weights * (labels.double() - predictions.double()).abs()).sum(dim=-1), WEIGHTED_NUM_SAMPES: weights.sum(dim=-1)}


class MAEMetricComputation(SumStatesComputation):
    STATES = (ERROR_SUM, WEIGHTED_NUM_SAMPES)

    def _states(self, labels, predictions, weights, **kwargs):
        return get_mae_states(labels, predictions, weights)

    def _values(self, s):
        return [(MetricName.MAE, compute_mae(s[ERROR_SUM], s[WEIGHTED_NUM_SAMPES]))]


class MAEMetric(RecMetric):
    _namespace = MetricNamespace.MAE
    _computation_class = MAEMetricComputation
