"""Normalized entropy: cross entropy of the predictions divided by the entropy of the base rate
(``torchrec/metrics/ne.py``).  Optionally also reports the plain log loss."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch

from torchrec_b200.metrics._sum_states import SumStatesComputation
from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace
from torchrec_b200.metrics.rec_metric import RecMetric


def compute_cross_entropy(labels: torch.Tensor, predictions: torch.Tensor, weights: torch.Tensor, eta: float) -> torch.Tensor:
    """Per-example weighted binary cross entropy in bits, predictions clamped to ``[eta, 1-eta]``."""
    p = predictions.double().clamp(min=eta, max=1 - eta)
    return -weights * (labels * torch.log2(p) + (1.0 - labels) * torch.log2(1.0 - p))


def base_rate_entropy(pos: torch.Tensor, neg: torch.Tensor, n: torch.Tensor, eta: float) -> torch.Tensor:
    """Total entropy (bits) of always predicting the positive rate."""
    mean = (pos / n.double().clamp(min=eta)).clamp(min=eta, max=1 - eta)
    return -pos * torch.log2(mean) - neg * torch.log2(1.0 - mean)


def compute_ne(ce_sum: torch.Tensor, weighted_num_samples: torch.Tensor, pos_labels: torch.Tensor, neg_labels: torch.Tensor, eta: float,
               allow_missing_label_with_zero_weight: bool = False) -> torch.Tensor:
    if allow_missing_label_with_zero_weight and not bool(weighted_num_samples.all()):
        return torch.full_like(ce_sum, eta)
    return ce_sum / base_rate_entropy(pos_labels, neg_labels, weighted_num_samples, eta)


def compute_logloss(ce_sum: torch.Tensor, pos_labels: torch.Tensor, neg_labels: torch.Tensor, eta: float) -> torch.Tensor:
    # same unit as the cross entropy sum (bits), per unit of label weight
    return ce_sum / (pos_labels + neg_labels).double().clamp(min=eta)


def get_ne_states(labels: torch.Tensor, predictions: torch.Tensor, weights: torch.Tensor, eta: float) -> Dict[str, torch.Tensor]:
    ce = compute_cross_entropy(labels, predictions, weights, eta)
    return {
        "cross_entropy_sum": ce.sum(dim=-1),
        "weighted_num_samples": weights.sum(dim=-1),
        "pos_labels": (weights * labels).sum(dim=-1),
        "neg_labels": (weights * (1.0 - labels)).sum(dim=-1),
    }


class NEMetricComputation(SumStatesComputation):
    STATES = ("cross_entropy_sum", "weighted_num_samples", "pos_labels", "neg_labels")

    def __init__(self, *args: Any, include_logloss: bool = False, allow_missing_label_with_zero_weight: bool = False, **kwargs: Any) -> None:
        self._include_logloss = include_logloss
        self._allow_missing = allow_missing_label_with_zero_weight
        super().__init__(*args, **kwargs)
        self.eta = 1e-12

    def _states(self, labels, predictions, weights, **kwargs):
        return get_ne_states(labels, predictions, weights, self.eta)

    def _values(self, s):
        out = [(MetricName.NE, compute_ne(s["cross_entropy_sum"], s["weighted_num_samples"], s["pos_labels"], s["neg_labels"], self.eta, self._allow_missing))]
        if self._include_logloss:
            out.append((MetricName.LOG_LOSS, compute_logloss(s["cross_entropy_sum"], s["pos_labels"], s["neg_labels"], self.eta)))
        return out


class NEMetric(RecMetric):
    _namespace = MetricNamespace.NE
    _computation_class = NEMetricComputation
