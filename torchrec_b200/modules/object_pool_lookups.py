"""Storage back ends of the object pools.

``TensorLookup`` keeps ``[pool_size, dim]`` rows; ``TensorJaggedIndexSelectLookup`` keeps, per id, one jagged row per feature in a
padded ``[pool_size, sum(capacity)]`` block plus ``[pool_size, F]`` lengths, and answers with a feature-major ``JaggedTensor``.  The
``UVMCaching*`` names are kept for API parity: with 180 GB of HBM per GPU the pools stay device resident, so they are the same
classes.  Counterpart of ``torchrec/modules/object_pool_lookups.py:29-762``."""
from __future__ import annotations

import abc
from typing import Dict, Iterator, List, Optional, Tuple

import torch

from torchrec_b200.ops import sparse_ops as sops
from torchrec_b200.sparse.jagged_tensor import JaggedTensor


class TensorPoolLookup(abc.ABC, torch.nn.Module):
    def __init__(self, pool_size: int, dim: int, dtype: torch.dtype, device: torch.device) -> None:
        super().__init__()
        self._pool_size, self._dim, self._dtype, self._device = pool_size, dim, dtype, device
        self._pool_init_device = device

    @abc.abstractmethod
    def lookup(self, ids: torch.Tensor) -> torch.Tensor: ...

    @abc.abstractmethod
    def update(self, ids: torch.Tensor, values: torch.Tensor) -> None: ...

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return self.lookup(ids)

    @abc.abstractmethod
    def states_to_register(self) -> Iterator[Tuple[str, torch.Tensor]]: ...

    @abc.abstractmethod
    def set_state(self, loaded_values: torch.Tensor) -> None: ...


class TensorLookup(TensorPoolLookup):
    def __init__(self, pool_size: int, dim: int, dtype: torch.dtype, device: torch.device, enable_uvm: bool = False) -> None:
        super().__init__(pool_size, dim, dtype, device)
        self._enable_uvm = enable_uvm  # accepted for parity; rows stay in device memory
        self._pool = torch.zeros(pool_size, dim, dtype=dtype, device=device)

    def lookup(self, ids: torch.Tensor) -> torch.Tensor:
        return self._pool.index_select(0, ids.to(self._pool.device).long())

    def update(self, ids: torch.Tensor, values: torch.Tensor) -> None:
        self._pool.index_copy_(0, ids.to(self._pool.device).long(), values.to(device=self._pool.device, dtype=self._pool.dtype))

    def set_state(self, loaded_values: torch.Tensor) -> None:
        self._pool.copy_(loaded_values)

    def states_to_register(self) -> Iterator[Tuple[str, torch.Tensor]]:
        yield "_pool", self._pool


class KeyedJaggedTensorPoolLookup(abc.ABC, torch.nn.Module):
    """``lookup(ids)`` -> ``JaggedTensor`` whose lengths are feature-major ``[F * len(ids)]``; ``update(ids, JaggedTensor)`` takes
    the same layout."""

    def __init__(self, pool_size: int, feature_max_lengths: Dict[str, int], is_weighted: bool, device: torch.device) -> None:
        super().__init__()
        self._pool_size, self._device, self._is_weighted = pool_size, device, is_weighted
        self._feature_max_lengths = dict(feature_max_lengths)
        self._caps: List[int] = list(feature_max_lengths.values())
        self._total_lengths = sum(self._caps)
        starts, acc = [], 0
        for c in self._caps:
            starts.append(acc)
            acc += c
        self._starts = starts

    @abc.abstractmethod
    def lookup(self, ids: torch.Tensor) -> JaggedTensor: ...

    @abc.abstractmethod
    def update(self, ids: torch.Tensor, values: JaggedTensor) -> None: ...

    def forward(self, ids: torch.Tensor) -> JaggedTensor:
        return self.lookup(ids)

    @abc.abstractmethod
    def states_to_register(self) -> Iterator[Tuple[str, torch.Tensor]]: ...


class TensorJaggedIndexSelectLookup(KeyedJaggedTensorPoolLookup):
    def __init__(self, pool_size: int, values_dtype: torch.dtype, feature_max_lengths: Dict[str, int], is_weighted: bool, device: torch.device) -> None:
        super().__init__(pool_size, feature_max_lengths, is_weighted, device)
        self._values = torch.zeros(pool_size, self._total_lengths, dtype=values_dtype, device=device)
        self._key_lengths = torch.zeros(pool_size, len(self._caps), dtype=torch.int64, device=device)
        self._weights = torch.zeros(pool_size, self._total_lengths if is_weighted else 0, dtype=torch.float32, device=device)

    def _pick(self, rows: torch.Tensor, lens: torch.Tensor) -> torch.Tensor:
        out = []
        for f, cap in enumerate(self._caps):
            block = rows[:, self._starts[f]: self._starts[f] + cap]
            out.append(block[torch.arange(cap, device=block.device).unsqueeze(0) < lens[:, f: f + 1]])
        return torch.cat(out) if out else rows.new_zeros(0)

    def lookup(self, ids: torch.Tensor) -> JaggedTensor:
        ids = ids.to(self._values.device).long()
        lens = self._key_lengths.index_select(0, ids)
        values = self._pick(self._values.index_select(0, ids), lens)
        weights = self._pick(self._weights.index_select(0, ids), lens) if self._is_weighted else None
        return JaggedTensor(values=values, weights=weights, lengths=lens.t().reshape(-1))

    def update(self, ids: torch.Tensor, values: JaggedTensor) -> None:
        ids = ids.to(self._values.device).long()
        B, F = ids.numel(), len(self._caps)
        lens = values.lengths().view(F, B).to(self._values.device)
        offsets = torch.cat([lens.new_zeros(1), lens.reshape(-1).cumsum(0)])
        for f, cap in enumerate(self._caps):
            lo, hi = int(offsets[f * B]), int(offsets[(f + 1) * B])
            seg_off = offsets[f * B: (f + 1) * B + 1] - lo
            v = values.values()[lo:hi].to(self._values.device)
            dense = sops.jagged_to_padded_dense(v, seg_off, cap, 0) if v.numel() else self._values.new_zeros(B, cap)
            self._values[ids, self._starts[f]: self._starts[f] + cap] = dense.to(self._values.dtype)
            if self._is_weighted and values.weights_or_none() is not None:
                w = values.weights()[lo:hi].to(self._values.device)
                self._weights[ids, self._starts[f]: self._starts[f] + cap] = sops.jagged_to_padded_dense(w, seg_off, cap, 0.0) if w.numel() else self._weights.new_zeros(B, cap)
            self._key_lengths[ids, f] = lens[f].clamp(max=cap)

    def states_to_register(self) -> Iterator[Tuple[str, torch.Tensor]]:
        yield "values", self._values
        yield "key_lengths", self._key_lengths
        if self._is_weighted:
            yield "weights", self._weights


# device-resident on this hardware: same classes under the cache-backed names
UVMCachingInt64Lookup = TensorJaggedIndexSelectLookup
UVMCachingInt32Lookup = TensorJaggedIndexSelectLookup
UVMCachingFloatLookup = TensorLookup
