"""Shared base for metrics that need the raw examples (AUC family): predictions / labels / weights of the last
``window_size`` examples are kept as lists of ``[n_tasks, n]`` tensors; ``compute`` gathers them from all ranks."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch

from torchrec_b200.metrics.metrics_namespace import MetricNameBase, MetricPrefix
from torchrec_b200.metrics.rec_metric import MetricComputationReport, RecMetricComputation, RecMetricException

PREDICTIONS = "predictions"
LABELS = "labels"
WEIGHTS = "weights"


class ListStatesComputation(RecMetricComputation):
    EXTRA: Tuple[str, ...] = ()  # extra per-example tensors taken from kwargs (e.g. grouping keys)

    def __init__(self, *args: Any, **kwargs: Any) -> None:
        super().__init__(*args, **kwargs)
        self._num_samples = 0
        for name in (PREDICTIONS, LABELS, WEIGHTS) + self.EXTRA:
            self._add_state(name, [], add_window_state=False, dist_reduce_fx="cat", persistent=False)

    def _extra(self, name: str, labels: torch.Tensor, kwargs: Dict[str, Any]) -> torch.Tensor:
        v = kwargs.get(name)
        if v is None:
            raise RecMetricException(f"{type(self).__name__} needs '{name}' in update()")
        return v.view(labels.shape[0], -1) if v.dim() <= 1 else v

    def update(self, *, predictions: Optional[torch.Tensor], labels: torch.Tensor, weights: Optional[torch.Tensor], **kwargs: Any) -> None:
        if predictions is None or weights is None:
            raise RecMetricException(f"Inputs 'predictions' and 'weights' should not be None for {type(self).__name__} update")
        items = {PREDICTIONS: predictions.double(), LABELS: labels.double(), WEIGHTS: weights.double()}
        for name in self.EXTRA:
            items[name] = self._extra(name, labels, kwargs)
        n = labels.shape[-1]
        for name, v in items.items():
            self._list_states[name].append(v.detach())
        self._num_samples += n
        # drop whole old updates while what remains still covers the window
        while len(self._list_states[LABELS]) > 1 and self._num_samples - self._list_states[LABELS][0].shape[-1] >= self._window_size:
            self._num_samples -= self._list_states[LABELS][0].shape[-1]
            for name in items:
                self._list_states[name].pop(0)

    def _cat(self, name: str) -> Optional[torch.Tensor]:
        lst = self._list_states[name]
        if not lst:
            return None
        t = torch.cat(lst, dim=-1)
        return t[..., -self._window_size:] if (self._window_size > 0 and t.shape[-1] > self._window_size and not self._gathered(name)) else t

    def _gathered(self, name: str) -> bool:
        return False

    def reset(self) -> None:
        super().reset()
        self._num_samples = 0
