"""``TensorList``: an append-only list of tensors handed to the native parameter-store client in one call
(``contrib/dynamic_embedding/src/torchrec_dynamic_embedding/tensor_list.py:21``)."""
from __future__ import annotations

from typing import Iterator, List

import torch


class TensorList:
    def __init__(self, tensors: List[torch.Tensor]) -> None:
        self._tensors: List[torch.Tensor] = []
        for t in tensors:
            self.append(t)

    def append(self, tensor: torch.Tensor) -> None:
        if not isinstance(tensor, torch.Tensor):
            raise TypeError(f"expected a tensor, got {type(tensor).__name__}")
        self._tensors.append(tensor)

    def __len__(self) -> int:
        return len(self._tensors)

    def __getitem__(self, i: int) -> torch.Tensor:
        return self._tensors[i]

    def __iter__(self) -> Iterator[torch.Tensor]:
        return iter(self._tensors)

    def tolist(self) -> List[torch.Tensor]:
        return list(self._tensors)
