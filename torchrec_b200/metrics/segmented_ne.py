"""NE per segment: examples carry an integer group key, every group gets its own NE
(``torchrec/metrics/segmented_ne.py``).  Reported as ``..._segmented_ne_<group>``."""
from __future__ import annotations

from typing import Any, Dict, List, Tuple

import torch

from torchrec_b200.metrics._sum_states import SumStatesComputation
from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace, MetricPrefix
from torchrec_b200.metrics.ne import compute_cross_entropy, compute_ne
from torchrec_b200.metrics.rec_metric import MetricComputationReport, RecMetric, RecMetricException

PREDICTIONS = "predictions"
LABELS = "labels"
WEIGHTS = "weights"


def compute_ne_helper(ce_sum: torch.Tensor, weighted_num_samples: torch.Tensor, pos_labels: torch.Tensor, neg_labels: torch.Tensor,
                      eta: float) -> torch.Tensor:
    """NE of every (task, group) cell at once: cross entropy over the entropy of the cell's base rate."""
    return compute_ne(ce_sum, weighted_num_samples, pos_labels, neg_labels, eta)


def get_segemented_ne_states(labels: torch.Tensor, predictions: torch.Tensor, weights: torch.Tensor, grouping_keys: torch.Tensor, eta: float,
                             num_groups: int) -> Dict[str, torch.Tensor]:
    """Per-group sums of the four NE states, ``[n_tasks, num_groups]``, as four products with the one-hot matrix of the keys (the
    reference walks the distinct keys with a mask each, ``torchrec/metrics/segmented_ne.py:105-152``).  Keys outside
    ``[0, num_groups)`` fall into the nearest group."""
    keys = grouping_keys.view(-1).long().clamp(0, num_groups - 1)
    onehot = torch.nn.functional.one_hot(keys, num_groups).double()  # [n, G]
    ce = compute_cross_entropy(labels, predictions, weights, eta)
    w, l = weights.double(), labels.double()
    return {"cross_entropy_sum": ce @ onehot, "weighted_num_samples": w @ onehot, "pos_labels": (w * l) @ onehot, "neg_labels": (w * (1 - l)) @ onehot}


class SegmentedNEMetricComputation(SumStatesComputation):
    STATES = ("cross_entropy_sum", "weighted_num_samples", "pos_labels", "neg_labels")

    def __init__(self, *args: Any, include_logloss: bool = False, num_groups: int = 1, grouping_keys: str = "grouping_keys",
                 cast_keys_to_int: bool = False, **kwargs: Any) -> None:
        self._num_groups = num_groups
        self._grouping_keys = grouping_keys
        self._cast_keys_to_int = cast_keys_to_int
        self._include_logloss = include_logloss
        super().__init__(*args, **kwargs)
        self.eta = 1e-12

    def _state_shape(self, name: str) -> Tuple[int, ...]:
        return (self._n_tasks, self._num_groups)

    def _states(self, labels, predictions, weights, **kwargs):
        req = kwargs.get("required_inputs") or {}
        keys = req.get(self._grouping_keys)
        if keys is None:
            raise RecMetricException(f"Inputs 'predictions' and 'weights' and '{self._grouping_keys}' should not be None for NEMetricComputation update")
        if self._cast_keys_to_int:
            keys = keys.to(torch.int64)
        return get_segemented_ne_states(labels, predictions, weights, keys, self.eta, self._num_groups)

    def _compute(self) -> List[MetricComputationReport]:
        reports = []
        for prefix, get in ((MetricPrefix.LIFETIME, lambda n: getattr(self, n)), (MetricPrefix.WINDOW, self.get_window_state)):
            ne = compute_ne_helper(get("cross_entropy_sum"), get("weighted_num_samples"), get("pos_labels"), get("neg_labels"), self.eta)
            for g in range(self._num_groups):
                reports.append(MetricComputationReport(name=MetricName.SEGMENTED_NE, metric_prefix=prefix, value=ne[:, g], description="_" + str(g)))
        return reports


class SegmentedNEMetric(RecMetric):
    _namespace = MetricNamespace.SEGMENTED_NE
    _computation_class = SegmentedNEMetricComputation

    def __init__(self, *args: Any, **kwargs: Any) -> None:
        super().__init__(*args, **kwargs)
        self._required_inputs.add(kwargs.get("grouping_keys", "grouping_keys"))
