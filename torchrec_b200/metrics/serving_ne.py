"""NE for serving-time monitoring: same math as NE, also reports the number of examples seen
(``torchrec/metrics/serving_ne.py``)."""
from __future__ import annotations

import torch

from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace, MetricPrefix
from torchrec_b200.metrics.ne import NEMetricComputation, compute_ne
from torchrec_b200.metrics.rec_metric import MetricComputationReport, RecMetric


class ServingNEMetricComputation(NEMetricComputation):
    STATES = NEMetricComputation.STATES + ("num_examples",)

    def _states(self, labels, predictions, weights, **kwargs):
        s = super()._states(labels, predictions, weights)
        s["num_examples"] = torch.full((labels.shape[0],), float(labels.shape[-1]), dtype=torch.double, device=labels.device)
        return s

    def _values(self, s):
        return [(MetricName.NE, compute_ne(s["cross_entropy_sum"], s["weighted_num_samples"], s["pos_labels"], s["neg_labels"], self.eta, self._allow_missing))]

    def _compute(self):
        reports = super()._compute()
        reports.append(MetricComputationReport(name=MetricName.TOTAL_EXAMPLES, metric_prefix=MetricPrefix.DEFAULT, value=self.num_examples.detach()))
        return reports


class ServingNEMetric(RecMetric):
    _namespace = MetricNamespace.SERVING_NE
    _computation_class = ServingNEMetricComputation
