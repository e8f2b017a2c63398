"""Session-level precision (``torchrec/metrics/precision_session.py``); see ``recall_session``."""
from __future__ import annotations

from typing import Any

from torchrec_b200.metrics._sum_states import safe_div
from torchrec_b200.metrics.metrics_config import RecComputeMode
from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace
from torchrec_b200.metrics.rec_metric import RecMetric
from torchrec_b200.metrics.recall_session import _check_session_args, _SessionComputation


class PrecisionSessionMetricComputation(_SessionComputation):
    STATES = ("num_true_pos", "num_false_pos")

    def _states(self, labels, predictions, weights, **kwargs):
        labels, pred_pos = self._ranked(labels, predictions, kwargs)
        return {"num_true_pos": (weights * labels * pred_pos).sum(dim=-1), "num_false_pos": (weights * (1 - labels) * pred_pos).sum(dim=-1)}

    def _values(self, s):
        return [(MetricName.PRECISION_SESSION_LEVEL, safe_div(s["num_true_pos"], s["num_true_pos"] + s["num_false_pos"], default=float("nan")))]


class PrecisionSessionMetric(RecMetric):
    _namespace = MetricNamespace.PRECISION_SESSION_LEVEL
    _computation_class = PrecisionSessionMetricComputation

    def __init__(self, world_size, my_rank, batch_size, tasks, compute_mode=RecComputeMode.UNFUSED_TASKS_COMPUTATION, window_size=100,
                 fused_update_limit=0, **kwargs: Any) -> None:
        _check_session_args("precision", tasks, compute_mode, fused_update_limit)
        super().__init__(world_size, my_rank, batch_size, tasks, compute_mode=compute_mode, window_size=window_size,
                         fused_update_limit=fused_update_limit, **kwargs)
        for task, comp in zip(tasks, self._metrics_computations):
            comp._set_def(task.session_metric_def)
            self._required_inputs.add(task.session_metric_def.session_var_name)
