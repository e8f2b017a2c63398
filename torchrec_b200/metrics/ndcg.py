"""NDCG@k per session, averaged over sessions (``torchrec/metrics/ndcg.py``).  By default reports ``1 - NDCG`` so
that the curve decreases like a loss.  Sessions are given by a per-example session id (``required_inputs[session_key]``)."""
from __future__ import annotations

from typing import Any, List, Optional

import torch

from torchrec_b200.metrics._session import ranking_within_session
from torchrec_b200.metrics._sum_states import SumStatesComputation, safe_div
from torchrec_b200.metrics.metrics_namespace import MetricName, MetricNamespace
from torchrec_b200.metrics.rec_metric import RecMetric, RecMetricException

SUM_NDCG = "sum_ndcg"
NUM_SESSIONS = "num_sessions"
SESSION_KEY = "session_id"


def session_ndcg(predictions: torch.Tensor, labels: torch.Tensor, session: torch.Tensor, k: int = -1, exponential_gain: bool = False,
                 remove_single_length_sessions: bool = False, weights: Optional[torch.Tensor] = None):
    """Returns ``(sum over sessions of NDCG, number of sessions counted)`` for 1-D inputs."""
    p, l, s = predictions.view(-1).double(), labels.view(-1).double(), session.view(-1)
    uniq, inv, counts = torch.unique(s, return_inverse=True, return_counts=True)
    gain = torch.pow(2.0, l) - 1.0 if exponential_gain else l
    rank_pred = ranking_within_session(p, s).view(-1)
    rank_ideal = ranking_within_session(l, s).view(-1)
    kk = k if k is not None and k > 0 else int(counts.max()) if counts.numel() else 0
    disc_pred = torch.where(rank_pred < kk, 1.0 / torch.log2(rank_pred.double() + 2.0), torch.zeros_like(p))
    disc_ideal = torch.where(rank_ideal < kk, 1.0 / torch.log2(rank_ideal.double() + 2.0), torch.zeros_like(p))
    dcg = torch.zeros(uniq.numel(), dtype=torch.double, device=p.device).index_add_(0, inv, gain * disc_pred)
    idcg = torch.zeros(uniq.numel(), dtype=torch.double, device=p.device).index_add_(0, inv, gain * disc_ideal)
    ndcg = torch.where(idcg > 0, dcg / idcg.clamp(min=1e-30), torch.zeros_like(dcg))
    keep = idcg > 0
    if remove_single_length_sessions:
        keep = keep & (counts > 1)
    if weights is not None:
        w = torch.zeros(uniq.numel(), dtype=torch.double, device=p.device).index_add_(0, inv, weights.view(-1).double()) / counts
        ndcg = ndcg * w
    return (ndcg * keep).sum(), keep.sum().double()


class NDCGComputation(SumStatesComputation):
    STATES = (SUM_NDCG, NUM_SESSIONS)

    def __init__(self, *args: Any, exponential_gain: bool = False, session_key: str = SESSION_KEY, k: int = -1,
                 report_ndcg_as_decreasing_curve: bool = True, remove_single_length_sessions: bool = False,
                 scale_by_weights_tensor: bool = False, is_negative_task_mask: Optional[List[bool]] = None, **kwargs: Any) -> None:
        self._exponential_gain = exponential_gain
        self._session_key = session_key
        self._k = k
        self._decreasing = report_ndcg_as_decreasing_curve
        self._remove_single = remove_single_length_sessions
        self._scale_by_weights = scale_by_weights_tensor
        self._neg_mask = is_negative_task_mask
        super().__init__(*args, **kwargs)

    def _states(self, labels, predictions, weights, **kwargs):
        req = kwargs.get("required_inputs") or {}
        if self._session_key not in req:
            raise RecMetricException(f"{self._session_key} must be passed in required_inputs")
        session = req[self._session_key]
        sums, nums = [], []
        for t in range(labels.shape[0]):
            p = predictions[t]
            if self._neg_mask is not None and self._neg_mask[t]:
                p = 1.0 - p
            a, b = session_ndcg(p, labels[t], session, self._k, self._exponential_gain, self._remove_single, weights[t] if self._scale_by_weights else None)
            sums.append(a); nums.append(b)
        return {SUM_NDCG: torch.stack(sums), NUM_SESSIONS: torch.stack(nums)}

    def _values(self, s):
        v = safe_div(s[SUM_NDCG], s[NUM_SESSIONS])
        return [(MetricName.NDCG, 1.0 - v if self._decreasing else v)]


class NDCGMetric(RecMetric):
    _namespace = MetricNamespace.NDCG
    _computation_class = NDCGComputation

    def __init__(self, *args: Any, **kwargs: Any) -> None:
        super().__init__(*args, **kwargs)
        self._required_inputs.add(kwargs.get("session_key", SESSION_KEY))
