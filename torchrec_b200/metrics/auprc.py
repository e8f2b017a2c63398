"""Weighted area under the precision-recall curve over the window (``torchrec/metrics/auprc.py``)."""
from __future__ import annotations

from typing import Any, List

import torch

from torchrec_b200.metrics._list_states import LABELS, PREDICTIONS, WEIGHTS, ListStatesComputation
from torchrec_b200.metrics.auc import GROUPING_KEYS
from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace, MetricPrefix
from torchrec_b200.metrics.rec_metric import MetricComputationReport, RecMetric


def _compute_auprc_helper(predictions: torch.Tensor, labels: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    """Step-wise integral of precision over recall (average precision); ties share one curve point."""
    order = torch.argsort(predictions, descending=True, stable=True)
    p, l, w = predictions[order], labels[order], weights[order]
    cum_tp = torch.cumsum(w * l, 0)
    cum_all = torch.cumsum(w, 0)
    if p.numel() == 0 or cum_tp[-1] == 0:
        return torch.tensor(0.0, dtype=torch.double, device=predictions.device)
    last_of_tie = torch.ones_like(p, dtype=torch.bool)
    last_of_tie[:-1] = p[1:] != p[:-1]
    tp, tot = cum_tp[last_of_tie], cum_all[last_of_tie]
    precision = tp / tot.clamp(min=torch.finfo(torch.double).tiny)
    recall = tp / cum_tp[-1]
    d_recall = recall - torch.cat([recall.new_zeros(1), recall[:-1]])
    return (precision * d_recall).sum()


def compute_auprc(n_tasks: int, predictions: torch.Tensor, labels: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    return torch.stack([_compute_auprc_helper(predictions[t], labels[t], weights[t]) for t in range(n_tasks)])


def compute_auprc_per_group(n_tasks: int, predictions: torch.Tensor, labels: torch.Tensor, weights: torch.Tensor,
                            grouping_keys: torch.Tensor) -> torch.Tensor:
    """Mean over the groups of the per-group AUPRC, per task (``torchrec/metrics/auprc.py:98-141``); a leading placeholder example
    with key -1 is ignored."""
    keys = grouping_keys.view(-1)
    if keys.numel() != 0 and int(keys[0]) == -1:
        keys, predictions, labels, weights = keys[1:], predictions[:, 1:], labels[:, 1:], weights[:, 1:]
    groups = torch.unique(keys)
    if groups.numel() == 0:
        return torch.zeros(n_tasks, dtype=torch.double, device=predictions.device)
    return torch.stack([torch.stack([_compute_auprc_helper(predictions[t][keys == g], labels[t][keys == g], weights[t][keys == g]) for g in groups]).mean()
                        for t in range(n_tasks)])


class AUPRCMetricComputation(ListStatesComputation):
    def __init__(self, *args: Any, grouped_auprc: bool = False, **kwargs: Any) -> None:
        self._grouped = grouped_auprc
        if grouped_auprc:
            self.EXTRA = (GROUPING_KEYS,)
        super().__init__(*args, **kwargs)

    def _compute(self) -> List[MetricComputationReport]:
        p, l, w = self._cat(PREDICTIONS), self._cat(LABELS), self._cat(WEIGHTS)
        if p is None:
            v = torch.zeros(self._n_tasks, dtype=torch.double)
        elif self._grouped:
            v = compute_auprc_per_group(self._n_tasks, p, l, w, self._cat(GROUPING_KEYS)[0])
        else:
            v = compute_auprc(self._n_tasks, p, l, w)
        return [MetricComputationReport(name=MetricName.AUPRC, metric_prefix=MetricPrefix.WINDOW, value=v)]


class AUPRCMetric(RecMetric):
    _namespace = MetricNamespace.AUPRC
    _computation_class = AUPRCMetricComputation
