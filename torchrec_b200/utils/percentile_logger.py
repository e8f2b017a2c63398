"""Sliding-window percentile logger for latency-like samples (``torchrec/utils/percentile_logger.py``)."""
from __future__ import annotations

import logging
import threading
from collections import deque
from typing import Deque, Dict, Optional

logger = logging.getLogger(__name__)


class PercentileLogger:
    def __init__(self, metric_name: str, window_size: int = 1000, log_interval: int = 100) -> None:
        self.metric_name = metric_name
        self.window_size = window_size
        self.log_interval = log_interval
        self._samples: Deque[float] = deque(maxlen=window_size)
        self._count = 0
        self._lock = threading.Lock()

    def add(self, value: float) -> None:
        with self._lock:
            self._samples.append(float(value))
            self._count += 1
            due = self._count % self.log_interval == 0
        if due:
            self.log()

    def percentiles(self) -> Dict[str, float]:
        with self._lock:
            data = sorted(self._samples)
        if not data:
            return {}
        pick = lambda q: data[min(len(data) - 1, int(q * (len(data) - 1) + 0.5))]
        return {"p50": pick(0.50), "p90": pick(0.90), "p95": pick(0.95), "p99": pick(0.99), "max": data[-1], "count": float(len(data))}

    def log(self) -> None:
        p = self.percentiles()
        if p:
            logger.info("%s: " + ", ".join(f"{k}={v:.4g}" for k, v in p.items()), self.metric_name)
