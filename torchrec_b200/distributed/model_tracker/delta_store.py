"""Per-table store of touched ids, appended every batch and compacted (de-duplicated) on demand
(``torchrec/distributed/model_tracker/delta_store.py:70``)."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from torchrec_b200.distributed.model_tracker.types import DeltaRows, EmbdUpdateMode, IndexedLookup


def _compute_unique_rows(ids: List[torch.Tensor], states: Optional[List[torch.Tensor]], mode: EmbdUpdateMode) -> DeltaRows:
    """Unique ids over all lookups; for FIRST / LAST the state of the first / last occurrence of every id."""
    cat_ids = torch.cat(ids)
    if states is None or mode == EmbdUpdateMode.NONE:
        return DeltaRows(ids=torch.unique(cat_ids), states=None)
    cat_states = torch.cat(states)
    uniq, inverse = torch.unique(cat_ids, return_inverse=True)
    pos = torch.arange(cat_ids.numel(), device=cat_ids.device)
    if mode == EmbdUpdateMode.FIRST:
        pick = torch.full((uniq.numel(),), cat_ids.numel(), dtype=torch.long, device=cat_ids.device).scatter_reduce_(0, inverse, pos, "amin", include_self=True)
    else:
        pick = torch.full((uniq.numel(),), -1, dtype=torch.long, device=cat_ids.device).scatter_reduce_(0, inverse, pos, "amax", include_self=True)
    return DeltaRows(ids=uniq, states=cat_states[pick])


class DeltaStore:
    def __init__(self, embdUpdateMode: EmbdUpdateMode = EmbdUpdateMode.NONE) -> None:
        self.embdUpdateMode = embdUpdateMode
        self.per_fqn_lookups: Dict[str, List[IndexedLookup]] = {}

    def append(self, batch_idx: int, fqn: str, ids: torch.Tensor, states: Optional[torch.Tensor]) -> None:
        self.per_fqn_lookups.setdefault(fqn, []).append(IndexedLookup(batch_idx=batch_idx, ids=ids, states=states))

    def delete(self, up_to_idx: Optional[int] = None) -> None:
        """Drop lookups of batches ``< up_to_idx`` (all when None)."""
        if up_to_idx is None:
            self.per_fqn_lookups = {}
            return
        for fqn, lookups in self.per_fqn_lookups.items():
            self.per_fqn_lookups[fqn] = [l for l in lookups if l.batch_idx >= up_to_idx]

    def compact(self, start_idx: int, end_idx: int) -> None:
        """Merge the lookups of batches ``[start_idx, end_idx)`` of every table into one de-duplicated lookup."""
        assert start_idx < end_idx, f"start_idx {start_idx} must be smaller than end_idx {end_idx}"
        for fqn, lookups in self.per_fqn_lookups.items():
            inside = [l for l in lookups if start_idx <= l.batch_idx < end_idx]
            if len(inside) <= 1:
                continue
            rows = _compute_unique_rows([l.ids for l in inside], [l.states for l in inside] if inside[0].states is not None else None, self.embdUpdateMode)
            merged = IndexedLookup(batch_idx=start_idx, ids=rows.ids, states=rows.states)
            self.per_fqn_lookups[fqn] = [l for l in lookups if l.batch_idx < start_idx] + [merged] + [l for l in lookups if l.batch_idx >= end_idx]

    def get_delta(self, from_idx: int = 0) -> Dict[str, DeltaRows]:
        out: Dict[str, DeltaRows] = {}
        for fqn, lookups in self.per_fqn_lookups.items():
            sel = [l for l in lookups if l.batch_idx >= from_idx]
            if not sel:
                continue
            out[fqn] = _compute_unique_rows([l.ids for l in sel], [l.states for l in sel] if sel[0].states is not None else None, self.embdUpdateMode)
        return out
