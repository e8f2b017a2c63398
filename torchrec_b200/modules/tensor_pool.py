"""``TensorPool``: ``pool_size`` rows of ``dim`` values addressed by id (``torchrec/modules/tensor_pool.py``)."""
from __future__ import annotations

from typing import Optional

import torch

from torchrec_b200.modules.object_pool import ObjectPool


class TensorPool(ObjectPool[torch.Tensor]):
    def __init__(self, pool_size: int, dim: int, dtype: torch.dtype, device: Optional[torch.device] = None, loading_mode=None, enable_uvm: bool = False) -> None:
        super().__init__()
        self._pool_size = pool_size
        self._dim = dim
        self._dtype = dtype
        self._device = device if device is not None else torch.device("cpu")
        self.register_buffer("_pool", torch.zeros(pool_size, dim, dtype=dtype, device=self._device))

    @property
    def pool_size(self) -> int:
        return self._pool_size

    @property
    def dim(self) -> int:
        return self._dim

    @property
    def dtype(self) -> torch.dtype:
        return self._dtype

    @property
    def device(self) -> torch.device:
        return self._pool.device

    @property
    def pool(self) -> torch.Tensor:
        return self._pool

    def lookup(self, ids: torch.Tensor) -> torch.Tensor:
        return self._pool.index_select(0, ids.to(self._pool.device).long())

    def update(self, ids: torch.Tensor, values: torch.Tensor) -> None:
        assert values.dim() == 2 and values.shape[1] == self._dim and values.dtype == self._dtype
        self._pool.index_copy_(0, ids.to(self._pool.device).long(), values.to(self._pool.device))

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return self.lookup(ids)
