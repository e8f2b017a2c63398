"""NE with predictions recalibrated for negative down-sampling: ``p' = c p / (c p + 1 - p)``
(``torchrec/metrics/ne_with_recalibration.py``)."""
from __future__ import annotations

from typing import Any

import torch

from torchrec_b200.metrics.metrics_namespace import MetricNamespace
from torchrec_b200.metrics.ne import NEMetricComputation
from torchrec_b200.metrics.rec_metric import RecMetric


def recalibrate(predictions: torch.Tensor, coefficient: float) -> torch.Tensor:
    return coefficient * predictions / (coefficient * predictions - predictions + 1.0)


class RecalibratedNEMetricComputation(NEMetricComputation):
    def __init__(self, *args: Any, recalibration_coefficient: float = 1.0, **kwargs: Any) -> None:
        self._recalibration_coefficient = recalibration_coefficient
        super().__init__(*args, **kwargs)

    def _states(self, labels, predictions, weights, **kwargs):
        return super()._states(labels, recalibrate(predictions, self._recalibration_coefficient), weights)


class RecalibratedNEMetric(RecMetric):
    _namespace = MetricNamespace.RECALIBRATED_NE
    _computation_class = RecalibratedNEMetricComputation
