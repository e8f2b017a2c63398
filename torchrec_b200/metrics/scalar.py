"""Reports a scalar carried in ``labels`` (e.g. a loss): latest value and window mean (``torchrec/metrics/scalar.py``)."""
from __future__ import annotations

from typing import Any, List, Optional

import torch

from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace, MetricPrefix
from torchrec_b200.metrics.rec_metric import MetricComputationReport, RecMetric, RecMetricComputation


class ScalarMetricComputation(RecMetricComputation):
    def __init__(self, *args: Any, **kwargs: Any) -> None:
        super().__init__(*args, **kwargs)
        self._add_state("labels", torch.zeros(self._n_tasks, dtype=torch.double), add_window_state=True, dist_reduce_fx="mean", persistent=False)
        self._add_state("window_count", torch.zeros(self._n_tasks, dtype=torch.double), add_window_state=True, dist_reduce_fx="mean", persistent=False)

    def update(self, *, predictions: Optional[torch.Tensor], labels: torch.Tensor, weights: Optional[torch.Tensor], **kwargs: Any) -> None:
        n = labels.shape[-1]
        value = labels.double().mean(dim=-1)
        ones = torch.ones(self._n_tasks, dtype=torch.double, device=labels.device)
        self.labels.copy_(value)
        self.window_count.copy_(ones)
        self._aggregate_window_state("labels", value, n)
        self._aggregate_window_state("window_count", ones, n)

    def _compute(self) -> List[MetricComputationReport]:
        return [
            MetricComputationReport(name=MetricName.SCALAR, metric_prefix=MetricPrefix.LIFETIME, value=self.labels),
            MetricComputationReport(name=MetricName.SCALAR, metric_prefix=MetricPrefix.WINDOW,
                                    value=self.get_window_state("labels") / self.get_window_state("window_count").clamp(min=1.0)),
        ]


class ScalarMetric(RecMetric):
    _namespace = MetricNamespace.SCALAR
    _computation_class = ScalarMetricComputation
