"""Regression AUC: the fraction of example pairs that the predictions order like the labels
(``torchrec/metrics/rauc.py``): 1 - (inversions of the labels when sorted by prediction) / (number of pairs)."""
from __future__ import annotations

from typing import Any, List

import torch

from torchrec_b200.metrics._list_states import LABELS, PREDICTIONS, WEIGHTS, ListStatesComputation
from torchrec_b200.metrics.auc import GROUPING_KEYS
from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace, MetricPrefix
from torchrec_b200.metrics.rec_metric import MetricComputationReport, RecMetric


def _count_inversions(x: torch.Tensor) -> int:
    """Pairs i < j with x[i] > x[j], by merge counting on the host (n log n)."""
    a = x.tolist()
    n = len(a)
    tmp = [0.0] * n
    inv = 0
    width = 1
    while width < n:
        for lo in range(0, n, 2 * width):
            mid, hi = min(lo + width, n), min(lo + 2 * width, n)
            i, j, k = lo, mid, lo
            while i < mid and j < hi:
                if a[i] <= a[j]:
                    tmp[k] = a[i]; i += 1
                else:
                    tmp[k] = a[j]; j += 1
                    inv += mid - i
                k += 1
            while i < mid:
                tmp[k] = a[i]; i += 1; k += 1
            while j < hi:
                tmp[k] = a[j]; j += 1; k += 1
        a, tmp = tmp, a
        width *= 2
    return inv


def _compute_rauc_helper(predictions: torch.Tensor, labels: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    n = predictions.numel()
    if n < 2:
        return torch.tensor(0.5, dtype=torch.double)
    # sort by (prediction, label): ties in the prediction count as ordered correctly
    order = torch.argsort(labels, stable=True)
    order = order[torch.argsort(predictions[order], stable=True)]
    inv = _count_inversions(labels[order].cpu())
    return torch.tensor(1.0 - inv / (n * (n - 1) / 2.0), dtype=torch.double)


def compute_rauc(n_tasks: int, predictions: torch.Tensor, labels: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    return torch.stack([_compute_rauc_helper(predictions[t], labels[t], weights[t]) for t in range(n_tasks)])


def count_reverse_pairs_divide_and_conquer(input: List[float]) -> float:
    """Fraction of the pairs of ``input`` that are out of order (a later element smaller than an earlier one)."""
    n = len(input)
    if n < 2:
        return 0.0
    return _count_inversions(torch.as_tensor(input, dtype=torch.double)) / (n * (n - 1) / 2)


def _without_padding(keys: torch.Tensor, *per_task: torch.Tensor):
    """Drop the leading placeholder example (key -1) that an empty state list carries so that a sync never gathers nothing."""
    if keys.numel() != 0 and int(keys[0]) == -1:
        return (keys[1:],) + tuple(t[:, 1:] for t in per_task)
    return (keys,) + per_task


def compute_rauc_per_group(n_tasks: int, predictions, labels, weights, grouping_keys: torch.Tensor) -> torch.Tensor:
    """Mean over the groups of the per-group RAUC, per task; inputs ``[n_tasks, n]`` tensors or lists of such chunks
    (``torchrec/metrics/rauc.py:151-205``)."""
    p, l, w = (torch.cat(list(x), dim=-1) if isinstance(x, (list, tuple)) else x for x in (predictions, labels, weights))
    keys, p, l, w = _without_padding(grouping_keys.view(-1), p, l, w)
    groups = torch.unique(keys)
    if groups.numel() == 0:
        return torch.full((n_tasks,), 0.5, dtype=torch.double)
    return torch.stack([torch.stack([_compute_rauc_helper(p[t][keys == g], l[t][keys == g], w[t][keys == g]) for g in groups]).mean()
                        for t in range(n_tasks)])


class RAUCMetricComputation(ListStatesComputation):
    def __init__(self, *args: Any, grouped_rauc: bool = False, **kwargs: Any) -> None:
        self._grouped = grouped_rauc
        if grouped_rauc:
            self.EXTRA = (GROUPING_KEYS,)
        super().__init__(*args, **kwargs)

    def _compute(self) -> List[MetricComputationReport]:
        p, l, w = self._cat(PREDICTIONS), self._cat(LABELS), self._cat(WEIGHTS)
        if p is None:
            v = torch.full((self._n_tasks,), 0.5, dtype=torch.double)
        elif self._grouped:
            v = compute_rauc_per_group(self._n_tasks, p, l, w, self._cat(GROUPING_KEYS)[0])
        else:
            v = compute_rauc(self._n_tasks, p, l, w)
        return [MetricComputationReport(name=MetricName.RAUC, metric_prefix=MetricPrefix.WINDOW, value=v.to(p.device if p is not None else "cpu"))]


class RAUCMetric(RecMetric):
    _namespace = MetricNamespace.RAUC
    _computation_class = RAUCMetricComputation
