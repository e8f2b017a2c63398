"""Passes aggregated model outputs through the metric pipeline: lifetime and window mean of the predictions
(``torchrec/metrics/output.py``)."""
from __future__ import annotations

import torch

from torchrec_b200.metrics._sum_states import SumStatesComputation, safe_div
from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace
from torchrec_b200.metrics.rec_metric import RecMetric


class OutputMetricComputation(SumStatesComputation):
    STATES = ("latest_imp", "total_latest_imp")

    def _states(self, labels, predictions, weights, **kwargs):
        return {"latest_imp": predictions.double().sum(dim=-1), "total_latest_imp": torch.full((labels.shape[0],), float(labels.shape[-1]), dtype=torch.double, device=labels.device)}

    def _values(self, s):
        return [(MetricName.OUTPUT, safe_div(s["latest_imp"], s["total_latest_imp"]))]


class OutputMetric(RecMetric):
    _namespace = MetricNamespace.OUTPUT
    _computation_class = OutputMetricComputation
