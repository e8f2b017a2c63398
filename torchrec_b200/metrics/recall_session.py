"""Session-level recall: predictions ranked inside their session; the ``top_threshold`` highest count as positive
(``torchrec/metrics/recall_session.py:199-216``)."""
from __future__ import annotations

from typing import Any, List, Optional

import torch

from torchrec_b200.metrics._session import ranking_within_session
from torchrec_b200.metrics._sum_states import SumStatesComputation, safe_div
from torchrec_b200.metrics.metrics_config import RecComputeMode, RecTaskInfo, SessionMetricDef
from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace
from torchrec_b200.metrics.rec_metric import RecMetric, RecMetricException


class _SessionComputation(SumStatesComputation):
    def __init__(self, *args: Any, session_metric_def: Optional[SessionMetricDef] = None, **kwargs: Any) -> None:
        super().__init__(*args, **kwargs)
        self._set_def(session_metric_def)

    def _set_def(self, d: Optional[SessionMetricDef]) -> None:
        self.session_metric_def = d
        self.top_threshold = d.top_threshold if d is not None else None
        self.run_ranking_of_labels = d.run_ranking_of_labels if d is not None else False
        self.session_var_name = d.session_var_name if d is not None else None

    def _ranked(self, labels, predictions, kwargs):
        req = kwargs.get("required_inputs") or {}
        session = req.get(self.session_var_name, kwargs.get("session"))
        if session is None:
            raise RecMetricException(f"the session tensor '{self.session_var_name}' must be passed in required_inputs")
        pred_pos = (ranking_within_session(predictions, session) < self.top_threshold).double()
        if self.run_ranking_of_labels:
            labels = (ranking_within_session(labels, session) < self.top_threshold).double()
        return labels, pred_pos


class RecallSessionMetricComputation(_SessionComputation):
    STATES = ("num_true_pos", "num_false_neg")

    def _states(self, labels, predictions, weights, **kwargs):
        labels, pred_pos = self._ranked(labels, predictions, kwargs)
        return {"num_true_pos": (weights * labels * pred_pos).sum(dim=-1), "num_false_neg": (weights * labels * (1 - pred_pos)).sum(dim=-1)}

    def _values(self, s):
        return [(MetricName.RECALL_SESSION_LEVEL, safe_div(s["num_true_pos"], s["num_true_pos"] + s["num_false_neg"], default=float("nan")))]


def _check_session_args(name: str, tasks: List[RecTaskInfo], compute_mode, fused_update_limit) -> None:
    if compute_mode in (RecComputeMode.FUSED_TASKS_COMPUTATION, RecComputeMode.FUSED_TASKS_AND_STATES_COMPUTATION):
        raise RecMetricException(f"Fused computation is not supported for {name} session-level metrics")
    if fused_update_limit > 0:
        raise RecMetricException(f"Fused update is not supported for {name} session-level metrics")
    for task in tasks:
        if task.session_metric_def is None:
            raise RecMetricException("Please, specify the session metric definition")
        if task.session_metric_def.top_threshold is None:
            raise RecMetricException("Please, specify the top threshold")


class RecallSessionMetric(RecMetric):
    _namespace = MetricNamespace.RECALL_SESSION_LEVEL
    _computation_class = RecallSessionMetricComputation

    def __init__(self, world_size, my_rank, batch_size, tasks, compute_mode=RecComputeMode.UNFUSED_TASKS_COMPUTATION, window_size=100,
                 fused_update_limit=0, **kwargs: Any) -> None:
        _check_session_args("recall", tasks, compute_mode, fused_update_limit)
        super().__init__(world_size, my_rank, batch_size, tasks, compute_mode=compute_mode, window_size=window_size,
                         fused_update_limit=fused_update_limit, **kwargs)
        for task, comp in zip(tasks, self._metrics_computations):
            comp._set_def(task.session_metric_def)
            self._required_inputs.add(task.session_metric_def.session_var_name)
