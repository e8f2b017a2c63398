"""Parameter-server clients for the tables of a sharded module."""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from torchrec_b200.contrib.dynamic_embedding.utils import ensure_native


class PS:
    """Client for one table.  ``shards``: list of ``(row_start, col_start, row_size, col_size, [weight, state...])`` of the
    local shard tensors (views into the kernel's buffers, so fetched rows land directly in the lookup memory)."""

    def __init__(self, table_name: str, shards: List[Tuple[int, int, int, int, List[torch.Tensor]]], col_size: int, num_optimizer_states: int,
                 url: str, chunk_size: int = 8 * 1024) -> None:
        ensure_native()
        lst = torch.classes.trb_tde.LocalShardList()
        for rs, cs, rn, cn, tensors in shards:
            lst.append(rs, cs, rn, cn, list(tensors))
        self._impl = torch.classes.trb_tde.PS(table_name, lst, col_size, num_optimizer_states, url, chunk_size)

    def fetch(self, ids_to_fetch: torch.Tensor, time: int, init: bool = True, weight_init_min: float = -0.01, weight_init_max: float = 0.01):
        return self._impl.fetch(ids_to_fetch, time, init, weight_init_min, weight_init_max)

    def evict(self, ids_to_evict: torch.Tensor) -> None:
        self._impl.evict(ids_to_evict)


class PSCollection:
    """One ``PS`` per table of a sharded embedding module."""

    def __init__(self, path: str, plan: Dict[str, Tuple[int, int]], state_dict: Dict[str, torch.Tensor], url: str, ps_config: Optional[dict] = None) -> None:
        self._ps: Dict[str, PS] = {}
        cfg = ps_config or {}
        for table, (rows, dim) in plan.items():
            w = state_dict[f"{table}.weight"] if f"{table}.weight" in state_dict else state_dict[table]
            if hasattr(w, "local_shards"):
                shards = [(s.metadata.shard_offsets[0], s.metadata.shard_offsets[1], s.metadata.shard_sizes[0], s.metadata.shard_sizes[1], [s.tensor]) for s in w.local_shards()]
            else:
                shards = [(0, 0, w.shape[0], w.shape[1], [w])]
            self._ps[table] = PS(f"{path}.{table}", shards, dim, 0, url, cfg.get("chunk_size", 8 * 1024))

    def keys(self):
        return self._ps.keys()

    def __getitem__(self, table: str) -> PS:
        return self._ps[table]
