"""A detached copy of the metric states taken between updates, so that compute can run off the training thread
(``torchrec/metrics/metric_state_snapshot.py``)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional

from torchrec_b200.metrics.metric_module import RecMetricModule
from torchrec_b200.metrics.throughput import ThroughputMetric


@dataclass
class MetricStateSnapshot:
    metric_states: Dict[str, Any]
    throughput_metric: Optional[ThroughputMetric]

    @classmethod
    def from_metrics(cls, module: RecMetricModule) -> "MetricStateSnapshot":
        return cls(metric_states=module.get_pre_compute_states(), throughput_metric=module.throughput_metric)

    def restore(self, module: RecMetricModule) -> None:
        module.load_pre_compute_states(self.metric_states)
