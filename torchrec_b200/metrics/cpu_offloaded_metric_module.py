"""Metric module whose updates and computes run on a worker thread: the training thread only copies the model
outputs to pinned host memory and enqueues a job (async hooks of ``torchrec/metrics/metric_module.py:493``)."""
from __future__ import annotations

import concurrent.futures
import queue
import threading
from typing import Any, Dict, Optional

import torch

from torchrec_b200.metrics.metric_job_types import MetricComputeJob, MetricUpdateJob
from torchrec_b200.metrics.metric_module import MetricValue, RecMetricModule


class CPUOffloadedRecMetricModule(RecMetricModule):
    def __init__(self, *args: Any, update_queue_size: int = 100, **kwargs: Any) -> None:
        super().__init__(*args, **kwargs)
        self._queue: "queue.Queue[Any]" = queue.Queue(maxsize=update_queue_size)
        self._shutdown = threading.Event()
        self._worker = threading.Thread(target=self._run, name="metric-worker", daemon=True)
        self._worker.start()

    def update(self, model_out: Dict[str, torch.Tensor], **kwargs: Any) -> None:
        host: Dict[str, torch.Tensor] = {}
        event = None
        for k, v in model_out.items():
            if isinstance(v, torch.Tensor) and v.is_cuda:
                buf = torch.empty(v.shape, dtype=v.dtype, device="cpu", pin_memory=True)
                buf.copy_(v.detach(), non_blocking=True)
                host[k] = buf
            else:
                host[k] = v.detach() if isinstance(v, torch.Tensor) else v
        if torch.cuda.is_available() and any(isinstance(v, torch.Tensor) and v.is_cuda for v in model_out.values()):
            event = torch.cuda.Event()
            event.record()
        self._queue.put(MetricUpdateJob(host, event, kwargs))

    def async_compute(self) -> "concurrent.futures.Future[Dict[str, MetricValue]]":
        fut: "concurrent.futures.Future[Dict[str, MetricValue]]" = concurrent.futures.Future()
        self._queue.put(MetricComputeJob(fut))
        return fut

    def compute(self) -> Dict[str, MetricValue]:
        return self.async_compute().result()

    def _run(self) -> None:
        while not self._shutdown.is_set():
            try:
                job = self._queue.get(timeout=0.1)
            except queue.Empty:
                continue
            try:
                if isinstance(job, MetricUpdateJob):
                    if job.transfer_completed_event is not None:
                        job.transfer_completed_event.synchronize()
                    RecMetricModule.update(self, job.model_out, **job.kwargs)
                elif isinstance(job, MetricComputeJob):
                    job.future.set_result(RecMetricModule.compute(self))
            except Exception as e:  # deliver failures to the waiting caller
                if isinstance(job, MetricComputeJob):
                    job.future.set_exception(e)

    def shutdown(self) -> None:
        self._shutdown.set()
        self._worker.join(timeout=5)
