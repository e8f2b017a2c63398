"""Weighted ROC AUC over the window of raw examples, optionally averaged over groups
(``torchrec/metrics/auc.py``)."""
from __future__ import annotations

from typing import Any, List, Optional

import torch

from torchrec_b200.metrics._list_states import LABELS, PREDICTIONS, WEIGHTS, ListStatesComputation
from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace, MetricPrefix
from torchrec_b200.metrics.rec_metric import MetricComputationReport, RecMetric

GROUPING_KEYS = "grouping_keys"


def _compute_auc_helper(predictions: torch.Tensor, labels: torch.Tensor, weights: torch.Tensor, apply_bin: bool = False) -> torch.Tensor:
    """Trapezoid area under the weighted ROC curve of one task; ties in the predictions share one curve point."""
    order = torch.argsort(predictions, descending=True, stable=True)
    p, l, w = predictions[order], labels[order], weights[order]
    cum_tp = torch.cumsum(w * l, 0)
    cum_fp = torch.cumsum(w * (1.0 - l), 0)
    if p.numel() == 0 or cum_tp[-1] == 0 or cum_fp[-1] == 0:
        return torch.tensor(0.5, dtype=torch.double, device=predictions.device)
    last_of_tie = torch.ones_like(p, dtype=torch.bool)
    last_of_tie[:-1] = p[1:] != p[:-1]
    tp = torch.cat([cum_tp.new_zeros(1), cum_tp[last_of_tie]])
    fp = torch.cat([cum_fp.new_zeros(1), cum_fp[last_of_tie]])
    return torch.trapz(tp, fp) / (cum_tp[-1] * cum_fp[-1])


def compute_auc(n_tasks: int, predictions: torch.Tensor, labels: torch.Tensor, weights: torch.Tensor, apply_bin: bool = False) -> torch.Tensor:
    return torch.stack([_compute_auc_helper(predictions[t], labels[t], weights[t], apply_bin) for t in range(n_tasks)])


def compute_auc_per_group(n_tasks: int, predictions: torch.Tensor, labels: torch.Tensor, weights: torch.Tensor, grouping_keys: torch.Tensor) -> torch.Tensor:
    """Unweighted mean of the per-group AUCs."""
    out = []
    keys = grouping_keys.view(-1)
    for t in range(n_tasks):
        vals = [_compute_auc_helper(predictions[t][keys == g], labels[t][keys == g], weights[t][keys == g]) for g in torch.unique(keys)]
        out.append(torch.stack(vals).mean() if vals else torch.tensor(0.5, dtype=torch.double))
    return torch.stack(out)


class AUCMetricComputation(ListStatesComputation):
    def __init__(self, *args: Any, grouped_auc: bool = False, apply_bin: bool = False, **kwargs: Any) -> None:
        self._grouped_auc = grouped_auc
        self._apply_bin = apply_bin
        if grouped_auc:
            self.EXTRA = (GROUPING_KEYS,)
        super().__init__(*args, **kwargs)

    def _compute(self) -> List[MetricComputationReport]:
        p, l, w = self._cat(PREDICTIONS), self._cat(LABELS), self._cat(WEIGHTS)
        if p is None:
            v = torch.full((self._n_tasks,), 0.5, dtype=torch.double)
        elif self._grouped_auc:
            v = compute_auc_per_group(self._n_tasks, p, l, w, self._cat(GROUPING_KEYS)[0])
        else:
            v = compute_auc(self._n_tasks, p, l, w, self._apply_bin)
        return [MetricComputationReport(name=MetricName.AUC, metric_prefix=MetricPrefix.WINDOW, value=v)]


class AUCMetric(RecMetric):
    _namespace = MetricNamespace.AUC
    _computation_class = AUCMetricComputation

    def __init__(self, *args: Any, **kwargs: Any) -> None:
        super().__init__(*args, **kwargs)
        if kwargs.get("grouped_auc"):
            self._required_inputs.add(GROUPING_KEYS)
