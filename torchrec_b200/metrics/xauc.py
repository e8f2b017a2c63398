"""XAUC: weighted fraction of example pairs (inside one update) ordered alike by prediction and label
(``torchrec/metrics/xauc.py:26-68``)."""
from __future__ import annotations

from typing import Dict

import torch

from torchrec_b200.metrics._sum_states import SumStatesComputation, safe_div
from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace
from torchrec_b200.metrics.rec_metric import RecMetric


def compute_error_sum(labels: torch.Tensor, predictions: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    p, l, w = predictions.double(), labels.double(), weights.double()
    dp = torch.sign(p.unsqueeze(-1) - p.unsqueeze(-2))
    dl = torch.sign(l.unsqueeze(-1) - l.unsqueeze(-2))
    ww = w.unsqueeze(-1) * w.unsqueeze(-2)
    match = (dp == dl).double() * ww  # concordant pairs and pairs tied in both
    return torch.triu(match, diagonal=1).sum(dim=(-1, -2))


def compute_weighted_num_pairs(weights: torch.Tensor) -> torch.Tensor:
    w = weights.double()
    return torch.triu(w.unsqueeze(-1) * w.unsqueeze(-2), diagonal=1).sum(dim=(-1, -2))


def compute_xauc(error_sum: torch.Tensor, weighted_num_pairs: torch.Tensor) -> torch.Tensor:
    """Concordant pair weight over total pair weight; 0 where no pair was seen."""
    return safe_div(error_sum, weighted_num_pairs)


def get_xauc_states(labels: torch.Tensor, predictions: torch.Tensor, weights: torch.Tensor) -> Dict[str, torch.Tensor]:
    return {"error_sum": compute_error_sum(labels, predictions, weights), "weighted_num_pairs": compute_weighted_num_pairs(weights)}


class XAUCMetricComputation(SumStatesComputation):
    STATES = ("error_sum", "weighted_num_pairs")

    def _states(self, labels, predictions, weights, **kwargs):
        return get_xauc_states(labels, predictions, weights)

    def _values(self, s):
        return [(MetricName.XAUC, compute_xauc(s["error_sum"], s["weighted_num_pairs"]))]


class XAUCMetric(RecMetric):
    _namespace = MetricNamespace.XAUC
    _computation_class = XAUCMetricComputation
