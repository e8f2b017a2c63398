"""Calibration of recalibrated predictions (``torchrec/metrics/calibration_with_recalibration.py``)."""
from __future__ import annotations

from typing import Any

from torchrec_b200.metrics.calibration import CalibrationMetricComputation
from torchrec_b200.metrics.metrics_namespace import MetricNamespace
from torchrec_b200.metrics.ne_with_recalibration import recalibrate
from torchrec_b200.metrics.rec_metric import RecMetric


class RecalibratedCalibrationMetricComputation(CalibrationMetricComputation):
    def __init__(self, *args: Any, recalibration_coefficient: float = 1.0, **kwargs: Any) -> None:
        self._recalibration_coefficient = recalibration_coefficient
        super().__init__(*args, **kwargs)

    def _states(self, labels, predictions, weights, **kwargs):
        return super()._states(labels, recalibrate(predictions, self._recalibration_coefficient), weights)


class RecalibratedCalibrationMetric(RecMetric):
    _namespace = MetricNamespace.RECALIBRATED_CALIBRATION
    _computation_class = RecalibratedCalibrationMetricComputation
