"""Mean squared error and its root (``torchrec/metrics/mse.py``); optionally R^2."""
from __future__ import annotations

from typing import Any, Dict

import torch

from torchrec_b200.metrics._sum_states import SumStatesComputation, safe_div
from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace
from torchrec_b200.metrics.rec_metric import RecMetric

ERROR_SUM = "error_sum"
WEIGHTED_NUM_SAMPES = "weighted_num_samples"
LABEL_SUM = "label_sum"
LABEL_SQUARED_SUM = "label_squared_sum"


def compute_mse(error_sum: torch.Tensor, weighted_num_samples: torch.Tensor) -> torch.Tensor:
    return safe_div(error_sum, weighted_num_samples)


def compute_rmse(error_sum: torch.Tensor, weighted_num_samples: torch.Tensor) -> torch.Tensor:
    return torch.sqrt(compute_mse(error_sum, weighted_num_samples))


def compute_r_squared(error_sum: torch.Tensor, weighted_num_samples: torch.Tensor, label_sum: torch.Tensor, label_squared_sum: torch.Tensor) -> torch.Tensor:
    total = label_squared_sum - safe_div(label_sum * label_sum, weighted_num_samples)
    return torch.where(total == 0, torch.zeros_like(total), 1.0 - safe_div(error_sum, total))


def get_mse_states(labels: torch.Tensor, predictions: torch.Tensor, weights: torch.Tensor) -> Dict[str, torch.Tensor]:
    d = labels.double() - predictions.double()
    return {
        ERROR_SUM: (weights * d * d).sum(dim=-1), WEIGHTED_NUM_SAMPES: weights.sum(dim=-1),
        LABEL_SUM: (weights * labels).sum(dim=-1), LABEL_SQUARED_SUM: (weights * labels.double() ** 2).sum(dim=-1),
    }


class MSEMetricComputation(SumStatesComputation):
    STATES = (ERROR_SUM, WEIGHTED_NUM_SAMPES, LABEL_SUM, LABEL_SQUARED_SUM)

    def __init__(self, *args: Any, include_r_squared: bool = False, **kwargs: Any) -> None:
        self._include_r_squared = include_r_squared
        super().__init__(*args, **kwargs)

    def _states(self, labels, predictions, weights, **kwargs):
        return get_mse_states(labels, predictions, weights)

    def _values(self, s):
        out = [(MetricName.MSE, compute_mse(s[ERROR_SUM], s[WEIGHTED_NUM_SAMPES])), (MetricName.RMSE, compute_rmse(s[ERROR_SUM], s[WEIGHTED_NUM_SAMPES]))]
        if self._include_r_squared:
            out.append((MetricName.R_SQUARED, compute_r_squared(s[ERROR_SUM], s[WEIGHTED_NUM_SAMPES], s[LABEL_SUM], s[LABEL_SQUARED_SUM])))
        return out


class MSEMetric(RecMetric):
    _namespace = MetricNamespace.MSE
    _computation_class = MSEMetricComputation
