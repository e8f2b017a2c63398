"""Work items of the CPU-offloaded metric path: a training thread enqueues updates / compute requests, a worker
applies them (``torchrec/metrics/metric_job_types.py``)."""
from __future__ import annotations

import concurrent.futures
from typing import Any, Dict

import torch


class MetricUpdateJob:
    """One batch of model outputs (already transferred to host memory) waiting to be applied to the metrics."""

    __slots__ = ["model_out", "transfer_completed_event", "kwargs"]

    def __init__(self, model_out: Dict[str, torch.Tensor], transfer_completed_event, kwargs: Dict[str, Any]) -> None:
        self.model_out = model_out
        self.transfer_completed_event = transfer_completed_event  # torch.cuda.Event or None
        self.kwargs = kwargs


class MetricComputeJob:
    """A request to compute; the result is delivered through ``future``."""

    __slots__ = ["future"]

    def __init__(self, future: "concurrent.futures.Future[Dict[str, Any]]") -> None:
        self.future = future


class SynchronizationMarker:
    """Queued by every rank before a compute so that all ranks compute after the same set of updates."""

    __slots__ = ["future"]

    def __init__(self, future: "concurrent.futures.Future[Dict[str, Any]]") -> None:
        self.future = future
