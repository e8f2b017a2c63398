"""Click-through rate: weighted positive labels over total weight (``torchrec/metrics/ctr.py``)."""
from __future__ import annotations

from typing import Dict

import torch

from torchrec_b200.metrics._sum_states import SumStatesComputation, safe_div
from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace
from torchrec_b200.metrics.rec_metric import RecMetric

CTR_NUM = "ctr_num"
CTR_DENOM = "ctr_denom"


def compute_ctr(ctr_num: torch.Tensor, ctr_denom: torch.Tensor) -> torch.Tensor:
    return safe_div(ctr_num, ctr_denom)


def get_ctr_states(labels: torch.Tensor, predictions: torch.Tensor, weights: torch.Tensor) -> Dict[str, torch.Tensor]:
    return {CTR_NUM: (labels * weights).sum(dim=-1), CTR_DENOM: weights.sum(dim=-1)}


class CTRMetricComputation(SumStatesComputation):
    STATES = (CTR_NUM, CTR_DENOM)

    def _states(self, labels, predictions, weights, **kwargs):
        return get_ctr_states(labels, predictions, weights)

    def _values(self, s):
        return [(MetricName.CTR, compute_ctr(s[CTR_NUM], s[CTR_DENOM]))]


class CTRMetric(RecMetric):
    _namespace = MetricNamespace.CTR
    _computation_class = CTRMetricComputation
