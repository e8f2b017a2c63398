"""Id transformers for all tables of an embedding collection: rewrites a KJT of global ids into cache slots and
keeps the parameter store in step (fetch rows of new ids, write evicted rows back)."""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from torchrec_b200.contrib.dynamic_embedding.id_transformer import IDTransformer
from torchrec_b200.contrib.dynamic_embedding.ps import PSCollection
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class IDTransformerCollection:
    def __init__(self, tables, eviction_config: Optional[dict] = None, transform_config: Optional[dict] = None,
                 ps_collection: Optional[PSCollection] = None) -> None:
        """``tables``: embedding (bag) configs; every table gets ``num_embeddings`` slots."""
        self._tables = list(tables)
        self._feature_to_table: Dict[str, int] = {}
        self._transformers: List[IDTransformer] = []
        self._table_names: List[str] = []
        for i, cfg in enumerate(self._tables):
            self._transformers.append(IDTransformer(cfg.num_embeddings, eviction_config, transform_config))
            self._table_names.append(cfg.name)
            for f in cfg.feature_names:
                if f in self._feature_to_table:
                    raise ValueError(f"feature {f} is used by two tables; dynamic embedding needs one table per feature")
                self._feature_to_table[f] = i
        self._ps_collection = ps_collection
        self._time = 0

    def _transform_ids(self, table_idx: int, global_ids: torch.Tensor) -> Tuple[torch.Tensor, List]:
        tr = self._transformers[table_idx]
        name = self._table_names[table_idx]
        gids = global_ids.to("cpu", torch.int64).contiguous()
        slots = torch.empty_like(gids)
        handles = []
        done = 0
        while done < gids.numel():
            r = tr.transform(gids[done:], slots[done:], self._time)
            if self._ps_collection is not None and r.ids_to_fetch.numel() > 0:
                handles.append(self._ps_collection[name].fetch(r.ids_to_fetch, self._time))
            done += r.num_transformed
            if not r.success:
                # out of slots: write the coldest rows back and free them, then continue with the rest
                for h in handles:
                    h.wait()
                handles = []
                evicted = tr.evict(max(tr._num_embedding // 8, 1))
                if evicted.numel() == 0:
                    raise RuntimeError(f"table {name}: one batch holds more distinct ids than the table has slots")
                if self._ps_collection is not None:
                    self._ps_collection[name].evict(evicted)
        return slots.to(global_ids.device), handles

    def transform(self, global_features: KeyedJaggedTensor) -> Tuple[KeyedJaggedTensor, List]:
        """Returns the KJT with cache slots as values and the fetch handles to wait on before the lookup."""
        self._time += 1
        values = global_features.values()
        out = torch.empty_like(values)
        handles: List = []
        lpk = global_features.length_per_key()
        start = 0
        for key, n in zip(global_features.keys(), lpk):
            if key in self._feature_to_table and n > 0:
                slots, hs = self._transform_ids(self._feature_to_table[key], values[start: start + n])
                out[start: start + n] = slots.to(out.dtype)
                handles.extend(hs)
            else:
                out[start: start + n] = values[start: start + n]
            start += n
        kjt = KeyedJaggedTensor(keys=global_features.keys(), values=out, lengths=global_features.lengths(), weights=global_features.weights_or_none(),
                                stride=global_features.stride())
        return kjt, handles

    def save(self) -> None:
        """Write every cached row back to the store."""
        if self._ps_collection is None:
            return
        for tr, name in zip(self._transformers, self._table_names):
            ids = tr.save()
            if ids.numel():
                self._ps_collection[name].evict(ids)
