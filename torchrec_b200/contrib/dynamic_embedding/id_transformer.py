"""Python face of the C++ id transformer."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from torchrec_b200.contrib.dynamic_embedding.utils import ensure_native


@dataclass
class TransformResult:
    success: bool
    num_transformed: int
    ids_to_fetch: torch.Tensor  # int64 [n, 2]: (global id, cache slot)


class IDTransformer:
    """``num_embedding`` cache slots for one table; ``eviction_config``: ``{"min_used_freq_power": int}``; ``transform_config``:
    ``{"type": "naive" | "cacheline"}`` selects the table layout of the native transformer (default ``"naive"``)."""

    def __init__(self, num_embedding: int, eviction_config: Optional[dict] = None, transform_config: Optional[dict] = None) -> None:
        ensure_native()
        cfg = eviction_config or {}
        self._num_embedding = num_embedding
        layout = str((transform_config or {}).get("type", "naive"))
        self._impl = torch.classes.trb_tde.IDTransformer(num_embedding, int(cfg.get("min_used_freq_power", 5)), layout)

    def transform(self, global_ids: torch.Tensor, cache_ids: torch.Tensor, time: int) -> TransformResult:
        r = self._impl.transform(global_ids, cache_ids, time)
        return TransformResult(bool(r.success), int(r.num_transformed), r.ids_to_fetch)

    def evict(self, num_to_evict: int) -> torch.Tensor:
        return self._impl.evict(num_to_evict)

    def save(self) -> torch.Tensor:
        return self._impl.save()

    def __len__(self) -> int:
        return int(self._impl.size())
