"""Calibration for serving-time monitoring, with the example count (``torchrec/metrics/serving_calibration.py``)."""
from __future__ import annotations

import torch

from torchrec_b200.metrics.calibration import CALIBRATION_DENOM, CALIBRATION_NUM, CalibrationMetricComputation, compute_calibration
from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace, MetricPrefix
from torchrec_b200.metrics.rec_metric import MetricComputationReport, RecMetric


class ServingCalibrationMetricComputation(CalibrationMetricComputation):
    STATES = CalibrationMetricComputation.STATES + ("num_examples",)

    def _states(self, labels, predictions, weights, **kwargs):
        s = super()._states(labels, predictions, weights)
        s["num_examples"] = torch.full((labels.shape[0],), float(labels.shape[-1]), dtype=torch.double, device=labels.device)
        return s

    def _values(self, s):
        return [(MetricName.CALIBRATION, compute_calibration(s[CALIBRATION_NUM], s[CALIBRATION_DENOM]))]

    def _compute(self):
        reports = super()._compute()
        reports.append(MetricComputationReport(name=MetricName.TOTAL_EXAMPLES, metric_prefix=MetricPrefix.DEFAULT, value=self.num_examples.detach()))
        return reports


class ServingCalibrationMetric(RecMetric):
    _namespace = MetricNamespace.SERVING_CALIBRATION
    _computation_class = ServingCalibrationMetricComputation
