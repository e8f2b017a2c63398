"""``KeyedJaggedTensorPool``: per id one jagged row per feature (e.g. a user's recent-item lists), stored densely with a
fixed capacity per (id, feature) and returned as a KJT (``torchrec/modules/keyed_jagged_tensor_pool.py``)."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from torchrec_b200.modules.object_pool import ObjectPool
from torchrec_b200.ops import sparse_ops as sops
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class KeyedJaggedTensorPool(ObjectPool[KeyedJaggedTensor]):
    def __init__(self, pool_size: int, feature_max_lengths: Dict[str, int], values_dtype: torch.dtype = torch.int64, is_weighted: bool = False,
                 device: Optional[torch.device] = None, enable_uvm: bool = False) -> None:
        super().__init__()
        self._pool_size = pool_size
        self._feature_max_lengths = dict(feature_max_lengths)
        self._keys = list(feature_max_lengths.keys())
        self._is_weighted = is_weighted
        self._device = device if device is not None else torch.device("cpu")
        self._total = sum(feature_max_lengths.values())
        starts, acc = [], 0
        for k in self._keys:
            starts.append(acc)
            acc += feature_max_lengths[k]
        self._starts = starts
        self.register_buffer("_values", torch.zeros(pool_size, self._total, dtype=values_dtype, device=self._device))
        self.register_buffer("_lengths", torch.zeros(pool_size, len(self._keys), dtype=torch.int64, device=self._device))
        if is_weighted:
            self.register_buffer("_weights", torch.zeros(pool_size, self._total, dtype=torch.float32, device=self._device))

    @property
    def pool_size(self) -> int:
        return self._pool_size

    @property
    def feature_max_lengths(self) -> Dict[str, int]:
        return self._feature_max_lengths

    def lookup(self, ids: torch.Tensor) -> KeyedJaggedTensor:
        ids = ids.to(self._values.device).long()
        B = ids.numel()
        lens = self._lengths.index_select(0, ids)  # [B, F]
        vals, wts = [], []
        rows = self._values.index_select(0, ids)
        wrows = self._weights.index_select(0, ids) if self._is_weighted else None
        for f, k in enumerate(self._keys):
            cap = self._feature_max_lengths[k]
            block = rows[:, self._starts[f]: self._starts[f] + cap]
            mask = torch.arange(cap, device=block.device).unsqueeze(0) < lens[:, f: f + 1]
            vals.append(block[mask])
            if wrows is not None:
                wts.append(wrows[:, self._starts[f]: self._starts[f] + cap][mask])
        return KeyedJaggedTensor(keys=self._keys, values=torch.cat(vals) if vals else self._values.new_zeros(0), lengths=lens.t().reshape(-1),
                                 weights=torch.cat(wts) if wts else None, stride=B)

    def update(self, ids: torch.Tensor, values: KeyedJaggedTensor) -> None:
        ids = ids.to(self._values.device).long()
        B = ids.numel()
        assert values.keys() == self._keys, "the KJT must carry the pool's features in the pool's order"
        lens = values.lengths().view(len(self._keys), B).to(self._lengths.device)
        jt = values.to_dict()
        for f, k in enumerate(self._keys):
            cap = self._feature_max_lengths[k]
            l = lens[f].clamp(max=cap)
            j = jt[k]
            dense = sops.jagged_to_padded_dense(j.values().to(self._values.device), j.offsets().to(self._values.device), cap, 0) if j.values().numel() else self._values.new_zeros(B, cap)
            self._values[ids, self._starts[f]: self._starts[f] + cap] = dense.to(self._values.dtype)
            if self._is_weighted and j.weights_or_none() is not None:
                wd = sops.jagged_to_padded_dense(j.weights().to(self._values.device), j.offsets().to(self._values.device), cap, 0.0)
                self._weights[ids, self._starts[f]: self._starts[f] + cap] = wd
            self._lengths[ids, f] = l

    def forward(self, ids: torch.Tensor) -> KeyedJaggedTensor:
        return self.lookup(ids)
