"""Multiclass recall@k for every k < n_classes: a sample counts at k when its label is among the k+1 highest-scored
classes (``torchrec/metrics/multiclass_recall.py:28-81``).  Predictions are ``[n_tasks, n, n_classes]``."""
from __future__ import annotations

from typing import Any, Dict, Tuple

import torch

from torchrec_b200.metrics._sum_states import SumStatesComputation
from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace
from torchrec_b200.metrics.rec_metric import RecMetric


def compute_true_positives_at_k(predictions: torch.Tensor, labels: torch.Tensor, weights: torch.Tensor, n_classes: int) -> torch.Tensor:
    ranks = torch.argsort(predictions, dim=-1, descending=True)
    hit = (ranks == labels.long().unsqueeze(-1)).double() * weights.double().unsqueeze(-1)  # [..., n, C]: hit at the rank of the label
    return torch.cumsum(hit.sum(dim=-2), dim=-1)


def compute_multiclass_recall_at_k(tp_at_k: torch.Tensor, total_weights: torch.Tensor) -> torch.Tensor:
    return tp_at_k / total_weights.unsqueeze(-1)


def get_multiclass_recall_states(predictions: torch.Tensor, labels: torch.Tensor, weights: torch.Tensor, n_classes: int) -> Dict[str, torch.Tensor]:
    return {"tp_at_k": compute_true_positives_at_k(predictions, labels, weights, n_classes), "total_weights": weights.double().sum(dim=-1)}


class MulticlassRecallMetricComputation(SumStatesComputation):
    STATES = ("tp_at_k", "total_weights")

    def __init__(self, *args: Any, number_of_classes: int = 2, **kwargs: Any) -> None:
        self._n_classes = number_of_classes
        super().__init__(*args, **kwargs)

    def _state_shape(self, name: str) -> Tuple[int, ...]:
        return (self._n_tasks, self._n_classes) if name == "tp_at_k" else (self._n_tasks,)

    def _states(self, labels, predictions, weights, **kwargs):
        if predictions.dim() == 2:  # [n, C] for a single task
            predictions = predictions.unsqueeze(0)
        return get_multiclass_recall_states(predictions, labels, weights, self._n_classes)

    def _values(self, s):
        return [(MetricName.MULTICLASS_RECALL, compute_multiclass_recall_at_k(s["tp_at_k"], s["total_weights"]))]


class MulticlassRecallMetric(RecMetric):
    _namespace = MetricNamespace.MULTICLASS_RECALL
    _computation_class = MulticlassRecallMetricComputation
