"""Training throughput: total / attempted examples and lifetime / window examples per second after a warm-up
(``torchrec/metrics/throughput.py:35-314``).  One ``update()`` per step; batch size is per rank and may follow a
schedule of ``BatchSizeStage``s."""
from __future__ import annotations

import math
import time
from collections import deque
from typing import Deque, Dict, List, Optional

import torch
from torch import nn

from torchrec_b200.metrics.metrics_config import BatchSizeStage, validate_batch_size_stages
from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace, MetricPrefix, compose_metric_key

MAX_WINDOW_TS: int = 2 * 60 * 60  # two hours


class ThroughputMetric(nn.Module):
    _namespace: MetricNamespace = MetricNamespace.THROUGHPUT

    def __init__(self, *, batch_size: int, world_size: int, window_seconds: int, warmup_steps: int = 100,
                 batch_size_stages: Optional[List[BatchSizeStage]] = None) -> None:
        super().__init__()
        if window_seconds < 1:
            raise ValueError("window_seconds must be at least 1 to give window throughput the minimum time window")
        if warmup_steps < 1:
            raise ValueError("warmup_steps must be at least 1 to give throughput a reasonable begin time.")
        window_seconds = min(window_seconds, MAX_WINDOW_TS)
        self._batch_size = batch_size
        self._world_size = world_size
        self._window_seconds = window_seconds
        self._warmup_steps = warmup_steps
        validate_batch_size_stages(batch_size_stages)
        self._batch_size_stages = list(batch_size_stages) if batch_size_stages else None
        self.register_buffer("total_examples", torch.tensor(0, dtype=torch.long))
        self.register_buffer("warmup_examples", torch.tensor(0, dtype=torch.long))
        self.register_buffer("time_lapse_after_warmup", torch.tensor(0, dtype=torch.double))
        self.register_buffer("attempt_examples", torch.tensor(0, dtype=torch.long))
        self.register_buffer("attempt_warmup_examples", torch.tensor(0, dtype=torch.long))
        self.register_buffer("attempt_time_lapse_after_warmup", torch.tensor(0, dtype=torch.double))
        self.register_buffer("_num_batch", torch.tensor(0, dtype=torch.long)) if self._batch_size_stages else None
        self._window_time_lapse_buffer: Deque[float] = deque(maxlen=MAX_WINDOW_TS)
        self._window_time_lapse = 0.0
        self._previous_ts = 0.0
        self._steps = 0
        self._lifetime_key = compose_metric_key(self._namespace, str(self._namespace), MetricName.THROUGHPUT, MetricPrefix.LIFETIME)
        self._window_key = compose_metric_key(self._namespace, str(self._namespace), MetricName.THROUGHPUT, MetricPrefix.WINDOW)
        self._attempt_key = compose_metric_key(self._namespace, str(self._namespace), MetricName.THROUGHPUT, MetricPrefix.ATTEMPT)
        self._total_examples_key = compose_metric_key(self._namespace, str(self._namespace), MetricName.TOTAL_EXAMPLES)
        self._attempt_examples_key = compose_metric_key(self._namespace, str(self._namespace), MetricName.ATTEMPT_EXAMPLES)
        self._batch_size_key = compose_metric_key(self._namespace, str(self._namespace), MetricName.BATCH_SIZE)

    def _current_batch_size(self) -> int:
        if not self._batch_size_stages:
            return self._batch_size
        nb = int(self._num_batch)
        while self._batch_size_stages and self._batch_size_stages[0].max_iters is not None and nb >= self._batch_size_stages[0].max_iters:
            if len(self._batch_size_stages) == 1:
                break
            self._batch_size_stages.pop(0)
        return self._batch_size_stages[0].batch_size

    def _check_window(self) -> None:
        while self._window_time_lapse > self._window_seconds and len(self._window_time_lapse_buffer) > 1:
            self._window_time_lapse -= self._window_time_lapse_buffer.popleft()

    def update(self) -> None:
        ts = time.monotonic()
        self._steps += 1
        bs = self._current_batch_size()
        if self._batch_size_stages is not None:
            self._num_batch += 1
        n = bs * self._world_size
        self.total_examples += n
        self.attempt_examples += n
        if self._steps <= self._warmup_steps:
            self.warmup_examples += n
            self.attempt_warmup_examples += n
            if self._steps == self._warmup_steps:
                self._previous_ts = ts
        else:
            lapse = ts - self._previous_ts
            self.time_lapse_after_warmup += lapse
            self.attempt_time_lapse_after_warmup += lapse
            self._window_time_lapse += lapse
            self._window_time_lapse_buffer.append(lapse)
            self._check_window()
            self._previous_ts = ts

    def compute(self) -> Dict[str, torch.Tensor]:
        ret: Dict[str, torch.Tensor] = {self._total_examples_key: self.total_examples, self._attempt_examples_key: self.attempt_examples}
        if self._steps > self._warmup_steps and (not math.isclose(float(self.time_lapse_after_warmup), 0) or not math.isclose(float(self.attempt_time_lapse_after_warmup), 0)):
            lifetime = (self.total_examples - self.warmup_examples) / self.time_lapse_after_warmup
            attempt = (self.attempt_examples - self.attempt_warmup_examples) / self.attempt_time_lapse_after_warmup
            window = len(self._window_time_lapse_buffer) * self._current_batch_size() * self._world_size / max(self._window_time_lapse, 1e-12)
            if not math.isclose(float(lifetime), 0):
                ret[self._lifetime_key] = torch.tensor(float(lifetime), dtype=torch.double)
            if not math.isclose(window, 0):
                ret[self._window_key] = torch.tensor(window, dtype=torch.double)
            if not math.isclose(float(attempt), 0):
                ret[self._attempt_key] = torch.tensor(float(attempt), dtype=torch.double)
        if self._batch_size_stages is not None:
            ret[self._batch_size_key] = torch.tensor(self._current_batch_size(), dtype=torch.int32)
        return ret
