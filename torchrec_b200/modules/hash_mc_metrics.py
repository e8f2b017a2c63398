"""Counters of the multi-probe hash (hit / insert / collision / eviction rates and table occupancy), accumulated on the device
and reported every ``frequency`` batches.  Counterpart of ``torchrec/modules/hash_mc_metrics.py`` (``ScalarLogger``)."""
from __future__ import annotations

import logging
from typing import Callable, Dict, Optional

import torch

logger: logging.Logger = logging.getLogger(__name__)


class ScalarLogger(torch.nn.Module):
    def __init__(self, name: str, zch_size: int, frequency: int, start_bucket: int = 0, disable_fallback: bool = False,
                 sink: Optional[Callable[[Dict[str, float]], None]] = None) -> None:
        super().__init__()
        self._name = name
        self._zch_size = zch_size
        self._frequency = frequency
        self._start_bucket = start_bucket
        self._disable_fallback = disable_fallback
        self._sink = sink
        self._batches = 0
        self._sums: Optional[torch.Tensor] = None  # [total, hit, insert, collision, evicted]
        self.last_report: Dict[str, float] = {}

    @torch.no_grad()
    def update(self, identities_0: torch.Tensor, identities_1: torch.Tensor, values: torch.Tensor, remapped_ids: torch.Tensor,
               evicted_emb_indices: Optional[torch.Tensor] = None, **_: object) -> None:
        """``identities_0/1``: the slot table before / after the batch; ``values``: the ids looked up; ``remapped_ids``: local slots."""
        n = values.numel()
        if n == 0:
            return
        valid = remapped_ids >= 0
        slot = remapped_ids.clamp(min=0)
        before = identities_0.view(-1).index_select(0, slot)
        after = identities_1.view(-1).index_select(0, slot)
        hit = valid & (before == values)
        stored = valid & (after == values)
        insert = stored & ~hit
        collision = ~stored
        ev = 0 if evicted_emb_indices is None else int((evicted_emb_indices >= 0).sum())
        row = torch.stack([torch.tensor(float(n), device=values.device), hit.sum().float(), insert.sum().float(), collision.sum().float(),
                           torch.tensor(float(ev), device=values.device)])
        self._sums = row if self._sums is None else self._sums + row

    @torch.no_grad()
    def forward(self, run_type: str, identities: torch.Tensor) -> None:
        self._batches += 1
        if self._frequency <= 0 or self._batches % self._frequency != 0 or self._sums is None:
            return
        total, hit, insert, collision, evicted = self._sums.tolist()
        total = max(total, 1.0)
        self.last_report = {
            f"{self._name}/{run_type}/hit_rate": hit / total,
            f"{self._name}/{run_type}/insert_rate": insert / total,
            f"{self._name}/{run_type}/collision_rate": collision / total,
            f"{self._name}/{run_type}/eviction_rate": evicted / total,
            f"{self._name}/{run_type}/occupancy": float((identities.view(-1) != -1).sum()) / max(self._zch_size, 1),
        }
        self._sums = None
        if self._sink is not None:
            self._sink(self.last_report)
        else:
            logger.info("zch %s bucket %d: %s", self._name, self._start_bucket, self.last_report)
