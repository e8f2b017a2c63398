"""NE that ignores the example weights (``torchrec/metrics/unweighted_ne.py``)."""
from __future__ import annotations

from typing import Dict

import torch

from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace
from torchrec_b200.metrics.ne import NEMetricComputation, compute_ne, get_ne_states
from torchrec_b200.metrics.rec_metric import RecMetric


def get_unweighted_ne_states(labels: torch.Tensor, predictions: torch.Tensor, weights: torch.Tensor, eta: float) -> Dict[str, torch.Tensor]:
    """The NE states with every example weighted 1 (``weights`` is accepted for a uniform signature and ignored)."""
    return get_ne_states(labels, predictions, torch.ones_like(predictions), eta)


class UnweightedNEMetricComputation(NEMetricComputation):
    def _states(self, labels, predictions, weights, **kwargs):
        return get_unweighted_ne_states(labels, predictions, weights, self.eta)

    def _values(self, s):
        out = super()._values(s)
        return [(MetricName.UNWEIGHTED_NE, out[0][1])] + out[1:]


class UnweightedNEMetric(RecMetric):
    _namespace = MetricNamespace.UNWEIGHTED_NE
    _computation_class = UnweightedNEMetricComputation
