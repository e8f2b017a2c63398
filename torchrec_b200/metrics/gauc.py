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


def to_3d(tensor_2d: torch.Tensor, seq_lengths: torch.Tensor, max_length: int) -> torch.Tensor:
    """Jagged rows ``[sum(seq_lengths), D]`` to a zero-padded ``[groups, max_length, D]`` block."""
    lengths = seq_lengths.view(-1).long()
    groups = lengths.numel()
    out = tensor_2d.new_zeros((groups, max_length, tensor_2d.shape[1]))
    gid = torch.repeat_interleave(torch.arange(groups, device=tensor_2d.device), lengths, output_size=tensor_2d.shape[0])
    start = torch.cumsum(lengths, 0) - lengths
    pos = torch.arange(tensor_2d.shape[0], device=tensor_2d.device) - start[gid]
    keep = pos < max_length
    out[gid[keep], pos[keep]] = tensor_2d[keep]
    return out


def compute_gauc_3d(predictions: torch.Tensor, labels: torch.Tensor, weights: torch.Tensor) -> Dict[str, torch.Tensor]:
    """Grouped AUC over zero-padded groups, all inputs ``[n_task, n_group, n_sample]``: padding carries weight 0, so it adds nothing
    to either class; a group counts when it has weight in both classes and its non-zero predictions are not all equal
    (``torchrec/metrics/gauc.py:24-91``).  Returns per-task ``auc_sum`` and ``num_samples``."""
    order = torch.argsort(predictions, dim=-1)
    l = torch.gather(labels, -1, order).double()
    w = torch.gather(weights, -1, order).double()
    neg_w = w * (1 - l)
    numer = (l * w * torch.cumsum(neg_w, dim=-1)).sum(-1)
    w_pos, w_neg = (l * w).sum(-1), neg_w.sum(-1)
    auc = numer / (w_pos * w_neg + 1e-10)
    flat = ((predictions == predictions[..., :1]) | (predictions == 0)).all(dim=-1)
    counted = (w_pos > 0) & (w_neg > 0) & ~flat
    return {"auc_sum": (auc * counted).sum(-1), "num_samples": counted.sum(-1)}


def get_auc_states(labels: torch.Tensor, predictions: torch.Tensor, weights: torch.Tensor, num_candidates: torch.Tensor) -> Dict[str, torch.Tensor]:
    """Per-task GAUC states from ``[n_task, n_sample]`` inputs whose samples are grouped by ``num_candidates``; computed on the jagged
    layout (one sort by (group, prediction)), without padding the groups to the longest one."""
    outs = [compute_gauc_jagged(predictions[t], labels[t], weights[t], num_candidates.view(-1)) for t in range(labels.shape[0])]
    return {"auc_sum": torch.stack([o["auc_sum"] for o in outs]), "num_samples": torch.stack([o["num_samples"] for o in outs])}


def compute_window_auc(auc: torch.Tensor, num_samples: torch.Tensor) -> Dict[str, torch.Tensor]:
    """Mean AUC over the counted groups; 0.5 when no group counted."""
    return {"gauc": (auc + 1e-9) / (num_samples + 2e-9), "num_samples": num_samples}


class GAUCMetricComputation(SumStatesComputation):
    STATES = ("auc_sum", "num_samples")

    def _states(self, labels, predictions, weights, **kwargs):
        nc = kwargs.get("num_candidates")
        if nc is None:
            nc = (kwargs.get("required_inputs") or {}).get("num_candidates")
        if nc is None:
            raise RecMetricException("GAUC needs 'num_candidates' (group sizes)")
        return get_auc_states(labels, predictions, weights, nc)

    def _values(self, s):
        return [(MetricName.GAUC, safe_div(s["auc_sum"], s["num_samples"])), (MetricName.GAUC_NUM_SAMPLES, s["num_samples"])]


class GAUCMetric(RecMetric):
    _namespace = MetricNamespace.GAUC
    _computation_class = GAUCMetricComputation

    def __init__(self, *args: Any, **kwargs: Any) -> None:
        super().__init__(*args, **kwargs)
        self._required_inputs.add("num_candidates")
