"""Measurement helpers of the ZCH benchmark: a skewed id stream and a probe that watches which raw id occupies which row.

``BenchmarkMCProbe.record(raw, remapped)`` keeps, per table row, the raw id last seen there.  A lookup whose row was last used by a
*different* raw id is a collision (two live ids share the row) or follows an eviction; both cost model quality, and both are
counted.  Counterpart of ``torchrec/distributed/benchmark/benchmark_zch/benchmark_zch_utils.py``."""
from __future__ import annotations

from typing import Dict, List

import torch


class ZipfIdStream:
    """Raw ids drawn from a fixed universe of ``distinct_ids`` 50-bit values with Zipf(alpha) popularity, one universe per feature."""

    def __init__(self, num_features: int, distinct_ids: int, alpha: float, input_hash_size: int, seed: int = 0) -> None:
        self._gen = torch.Generator().manual_seed(seed)
        self._universe = [torch.randint(0, input_hash_size, (distinct_ids,), generator=self._gen) for _ in range(num_features)]
        weights = 1.0 / torch.arange(1, distinct_ids + 1, dtype=torch.float64) ** alpha
        self._probs = (weights / weights.sum()).float()

    def draw(self, feature: int, n: int) -> torch.Tensor:
        return self._universe[feature][torch.multinomial(self._probs, n, replacement=True, generator=self._gen)]


class BenchmarkMCProbe:
    def __init__(self, table_names: List[str], zch_size: int, device: torch.device) -> None:
        self._owner: Dict[str, torch.Tensor] = {t: torch.full((zch_size,), -1, dtype=torch.int64, device=device) for t in table_names}
        self.lookups = 0
        self.conflicts = 0
        self.inserts = 0

    @torch.no_grad()
    def record(self, table: str, raw: torch.Tensor, remapped: torch.Tensor) -> None:
        owner = self._owner[table]
        raw, remapped = raw.to(owner.device).long(), remapped.to(owner.device).long()
        # judge each distinct raw id of the batch once
        uniq, first = torch.unique(raw, return_inverse=False, return_counts=False, sorted=True), None
        del first
        idx = torch.searchsorted(uniq, raw)
        slot = torch.empty_like(uniq).scatter_(0, idx, remapped)
        prev = owner[slot]
        self.lookups += int(uniq.numel())
        self.inserts += int((prev == -1).sum())
        self.conflicts += int(((prev != -1) & (prev != uniq)).sum())
        # ids of this batch that landed on the same row also conflict with each other
        order = torch.argsort(slot)
        s_sorted = slot[order]
        self.conflicts += int((s_sorted[1:] == s_sorted[:-1]).sum())
        owner[slot] = uniq

    def occupancy(self) -> float:
        used = sum(int((o != -1).sum()) for o in self._owner.values())
        return used / max(sum(o.numel() for o in self._owner.values()), 1)

    def summary(self) -> Dict[str, float]:
        return {"distinct_lookups": self.lookups, "inserts": self.inserts, "conflicts": self.conflicts,
                "collision_rate": self.conflicts / max(self.lookups, 1), "occupancy": self.occupancy()}
