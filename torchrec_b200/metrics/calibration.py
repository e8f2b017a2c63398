"""Calibration: sum of weighted predictions over sum of weighted labels (``torchrec/metrics/calibration.py``)."""
from __future__ import annotations

from typing import Dict

import torch

from torchrec_b200.metrics._sum_states import SumStatesComputation, safe_div
from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace
from torchrec_b200.metrics.rec_metric import RecMetric

CALIBRATION_NUM = "calibration_num"
CALIBRATION_DENOM = "calibration_denom"


def compute_calibration(calibration_num: torch.Tensor, calibration_denom: torch.Tensor) -> torch.Tensor:
    return safe_div(calibration_num, calibration_denom)


def get_calibration_states(labels: torch.Tensor, predictions: torch.Tensor, weights: torch.Tensor) -> Dict[str, torch.Tensor]:
    return {CALIBRATION_NUM: (predictions * weights).sum(dim=-1), CALIBRATION_DENOM: (labels * weights).sum(dim=-1)}


class CalibrationMetricComputation(SumStatesComputation):
    STATES = (CALIBRATION_NUM, CALIBRATION_DENOM)

    def _states(self, labels, predictions, weights, **kwargs):
        return get_calibration_states(labels, predictions, weights)

    def _values(self, s):
        return [(MetricName.CALIBRATION, compute_calibration(s[CALIBRATION_NUM], s[CALIBRATION_DENOM]))]


class CalibrationMetric(RecMetric):
    _namespace = MetricNamespace.CALIBRATION
    _computation_class = CalibrationMetricComputation
