"""Weighted average of an arbitrary named tensor of the model output (``torchrec/metrics/tensor_weighted_avg.py``).
The task's ``tensor_name`` selects the tensor from ``required_inputs``; ``weighted=False`` ignores the weights."""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch

from torchrec_b200.metrics._sum_states import SumStatesComputation
from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace
from torchrec_b200.metrics.rec_metric import RecMetric, RecMetricException
from torchrec_b200.metrics.weighted_avg import get_mean


class TensorWeightedAvgMetricComputation(SumStatesComputation):
    STATES = ("weighted_sum", "weighted_num_samples")
    NEEDS_PREDICTIONS = False

    def __init__(self, *args: Any, tensor_name: Optional[str] = None, weighted: bool = True, description: Optional[str] = None, **kwargs: Any) -> None:
        if tensor_name is None:
            raise RecMetricException("TensorWeightedAvgMetric requires tensor_name to be specified")
        self.tensor_name = tensor_name
        self.weighted = weighted
        super().__init__(*args, **kwargs)

    def _states(self, labels, predictions, weights, **kwargs):
        req = kwargs.get("required_inputs")
        if req is None or self.tensor_name not in req:
            raise RecMetricException(f"required_inputs must contain '{self.tensor_name}'")
        t = req[self.tensor_name]
        t = t.view(labels.shape[0], -1) if t.dim() <= 1 or t.shape != labels.shape else t
        w = weights if self.weighted else torch.ones_like(t, dtype=torch.float32)
        return {"weighted_sum": (t * w).sum(dim=-1), "weighted_num_samples": w.sum(dim=-1)}

    def _values(self, s):
        return [(MetricName.WEIGHTED_AVG, get_mean(s["weighted_sum"], s["weighted_num_samples"]))]


class TensorWeightedAvgMetric(RecMetric):
    _namespace = MetricNamespace.WEIGHTED_AVG
    _computation_class = TensorWeightedAvgMetricComputation

    def __init__(self, world_size, my_rank, batch_size, tasks, **kwargs: Any) -> None:
        # one computation per task, each bound to its task's tensor
        self._task_args = [(t.tensor_name, t.weighted) for t in tasks]
        super().__init__(world_size, my_rank, batch_size, tasks, tensor_name=tasks[0].tensor_name, weighted=tasks[0].weighted, **kwargs)
        for comp, (name, weighted) in zip(self._metrics_computations, self._task_args):
            if name is None:
                raise RecMetricException("TensorWeightedAvgMetric requires tensor_name on every task")
            comp.tensor_name, comp.weighted = name, weighted
            self._required_inputs.add(name)
