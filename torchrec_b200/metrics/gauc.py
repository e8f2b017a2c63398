"""Grouped AUC: AUC inside every group (e.g. per user), averaged over the groups that have both classes and
non-constant predictions (``torchrec/metrics/gauc.py:24-99``).  Groups are given by ``num_candidates`` (group sizes,
examples of a group are contiguous)."""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch

from torchrec_b200.metrics._sum_states import SumStatesComputation, safe_div
from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace, MetricPrefix
from torchrec_b200.metrics.rec_metric import MetricComputationReport, RecMetric, RecMetricException


def compute_gauc_jagged(predictions: torch.Tensor, labels: torch.Tensor, weights: torch.Tensor, num_candidates: torch.Tensor) -> Dict[str, torch.Tensor]:
    """1-D inputs; returns the sum of per-group AUCs and the number of groups that counted."""
    n = predictions.numel()
    gid = torch.repeat_interleave(torch.arange(num_candidates.numel(), device=predictions.device), num_candidates.long(), output_size=n)
    order = torch.argsort(predictions.double(), stable=True)
    order = order[torch.argsort(gid[order], stable=True)]  # by (group, prediction ascending)
    g, l, w, p = gid[order], labels[order].double(), weights[order].double(), predictions[order].double()
    neg_w = w * (1 - l)
    csum = torch.cumsum(neg_w, 0)
    G = num_candidates.numel()
    start = torch.zeros(G, dtype=torch.long, device=p.device)
    start[1:] = torch.cumsum(num_candidates.long(), 0)[:-1]
    base = torch.where(start > 0, csum[(start - 1).clamp(min=0)], torch.zeros(G, dtype=torch.double, device=p.device))
    cum_neg_in_group = csum - base[g]
    numer = torch.zeros(G, dtype=torch.double, device=p.device).index_add_(0, g, l * w * cum_neg_in_group)
    w_pos = torch.zeros(G, dtype=torch.double, device=p.device).index_add_(0, g, l * w)
    w_neg = torch.zeros(G, dtype=torch.double, device=p.device).index_add_(0, g, neg_w)
    auc = numer / (w_pos * w_neg + 1e-10)
    pmax = torch.full((G,), -float("inf"), dtype=torch.double, device=p.device).scatter_reduce_(0, g, p, "amax")
    pmin = torch.full((G,), float("inf"), dtype=torch.double, device=p.device).scatter_reduce_(0, g, p, "amin")
    mask = (w_pos > 0) & (w_neg > 0) & (pmax > pmin)
    return {"auc_sum": (auc * mask).sum(), "num_samples": mask.sum().double()}


class GAUCMetricComputation(SumStatesComputation):
    STATES = ("auc_sum", "num_samples")

    def _states(self, labels, predictions, weights, **kwargs):
        nc = kwargs.get("num_candidates")
        if nc is None:
            nc = (kwargs.get("required_inputs") or {}).get("num_candidates")
        if nc is None:
            raise RecMetricException("GAUC needs 'num_candidates' (group sizes)")
        outs = [compute_gauc_jagged(predictions[t], labels[t], weights[t], nc.view(-1)) for t in range(labels.shape[0])]
        return {"auc_sum": torch.stack([o["auc_sum"] for o in outs]), "num_samples": torch.stack([o["num_samples"] for o in outs])}

    def _values(self, s):
        return [(MetricName.GAUC, safe_div(s["auc_sum"], s["num_samples"])), (MetricName.GAUC_NUM_SAMPLES, s["num_samples"])]


class GAUCMetric(RecMetric):
    _namespace = MetricNamespace.GAUC
    _computation_class = GAUCMetricComputation

    def __init__(self, *args: Any, **kwargs: Any) -> None:
        super().__init__(*args, **kwargs)
        self._required_inputs.add("num_candidates")
