"""``ModelDeltaTracker``: hooks the sharded embedding modules of a model and records, per table, which rows every batch
touched (optionally with the looked-up embeddings), so that a consumer can publish or checkpoint only what changed
since it last asked (``torchrec/distributed/model_tracker/model_delta_tracker.py:39``)."""
from __future__ import annotations

from typing import Dict, List, Optional, Set

import torch
from torch import nn

from torchrec_b200.distributed.model_tracker.delta_store import DeltaStore
from torchrec_b200.distributed.model_tracker.types import DeltaRows, EmbdUpdateMode, TrackingMode
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

_MODE_MAP = {TrackingMode.ID_ONLY: EmbdUpdateMode.NONE, TrackingMode.EMBEDDING: EmbdUpdateMode.FIRST, TrackingMode.MOMENTUM_LAST: EmbdUpdateMode.LAST,
             TrackingMode.MOMENTUM_DIFF: EmbdUpdateMode.FIRST, TrackingMode.ROWWISE_ADAGRAD: EmbdUpdateMode.LAST}
DEFAULT_CONSUMER = "default"


class ModelDeltaTracker:
    def __init__(self, model: nn.Module, consumers: Optional[List[str]] = None, delete_on_read: bool = True, auto_compact: bool = False,
                 mode: TrackingMode = TrackingMode.ID_ONLY, fqns_to_skip: Optional[List[str]] = None) -> None:
        self._model = model
        self._consumers = consumers or [DEFAULT_CONSUMER]
        self._delete_on_read = delete_on_read
        self._auto_compact = auto_compact
        self._mode = mode
        self._fqns_to_skip: Set[str] = set(fqns_to_skip or [])
        self.store = DeltaStore(_MODE_MAP[mode])
        self.curr_batch_idx = 0
        self.curr_compact_index = 0
        self.per_consumer_batch_idx: Dict[str, int] = {c: 0 for c in self._consumers}
        self.feature_to_fqn: Dict[str, str] = {}
        self.tracked_modules: Dict[str, nn.Module] = {}
        self._discover(model)

    def _discover(self, model: nn.Module) -> None:
        """Sharded embedding modules expose ``post_lookup_tracker_fn``; map every feature to ``<module path>.<table>``."""
        from torchrec_b200.distributed.embedding_types import ShardedEmbeddingModule

        for path, m in model.named_modules():
            if isinstance(m, ShardedEmbeddingModule):
                if any(s in path for s in self._fqns_to_skip):
                    continue
                configs = getattr(m, "_embedding_bag_configs", None) or getattr(m, "_embedding_configs", [])
                for cfg in configs:
                    for f in cfg.feature_names:
                        self.feature_to_fqn[f] = f"{path}.{cfg.name}" if path else cfg.name
                self.tracked_modules[path] = m
                m.post_lookup_tracker_fn = self.record_lookup

    def step(self) -> None:
        """Call once per batch (after backward)."""
        self.curr_batch_idx += 1
        if self._auto_compact and self.curr_batch_idx - self.curr_compact_index > 1:
            self.store.compact(self.curr_compact_index, self.curr_batch_idx)

    def record_lookup(self, kjt: KeyedJaggedTensor, states: Optional[torch.Tensor], emb_module: Optional[nn.Module] = None, pooling=None) -> None:
        """Called by the sharded module after a lookup with the (post input-dist) ids and, for unpooled lookups, the rows."""
        lpk = kjt.length_per_key()
        ids = kjt.values()
        start = 0
        per_fqn_ids: Dict[str, List[torch.Tensor]] = {}
        per_fqn_states: Dict[str, List[torch.Tensor]] = {}
        want_states = self._mode != TrackingMode.ID_ONLY and states is not None and states.dim() == 2 and states.shape[0] == ids.numel()
        for key, n in zip(kjt.keys(), lpk):
            fqn = self.feature_to_fqn.get(key)
            if fqn is not None and n > 0:
                per_fqn_ids.setdefault(fqn, []).append(ids[start: start + n].detach())
                if want_states:
                    per_fqn_states.setdefault(fqn, []).append(states[start: start + n].detach())
            start += n
        for fqn, parts in per_fqn_ids.items():
            self.store.append(self.curr_batch_idx, fqn, torch.cat(parts), torch.cat(per_fqn_states[fqn]) if fqn in per_fqn_states else None)

    def get_unique_ids(self, consumer: Optional[str] = None) -> Dict[str, torch.Tensor]:
        return {fqn: rows.ids for fqn, rows in self.get_unique(consumer).items()}

    def get_unique(self, consumer: Optional[str] = None) -> Dict[str, DeltaRows]:
        """Rows touched since ``consumer`` last asked."""
        consumer = consumer or self._consumers[0]
        assert consumer in self.per_consumer_batch_idx, f"consumer {consumer} not present in {self._consumers}"
        from_idx = self.per_consumer_batch_idx[consumer]
        delta = self.store.get_delta(from_idx)
        self.per_consumer_batch_idx[consumer] = self.curr_batch_idx
        if self._delete_on_read:
            self.store.delete(up_to_idx=min(self.per_consumer_batch_idx.values()))
        self.curr_compact_index = self.curr_batch_idx
        return delta

    def fqn_to_feature_names(self) -> Dict[str, List[str]]:
        out: Dict[str, List[str]] = {}
        for f, fqn in self.feature_to_fqn.items():
            out.setdefault(fqn, []).append(f)
        return out

    def clear(self, consumer: Optional[str] = None) -> None:
        self.store.delete()
