"""Cached regrouping of ``KeyedTensor``s: the column permutation for a fixed set of groups is computed on the first call
and reused (``torchrec/modules/regroup.py:56,128``)."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
from torch import nn

from torchrec_b200.sparse.jagged_tensor import KeyedTensor


class PermuteMultiEmbedding(nn.Module):
    """Regroups several ``[B, sum D]`` tensors into ``len(groups)`` tensors by key; the gather index is cached per device."""

    def __init__(self, groups: List[List[str]]) -> None:
        super().__init__()
        self._groups = groups
        self._index: Optional[torch.Tensor] = None
        self._out_lengths: Optional[List[int]] = None

    def init_tensors(self, keys: List[List[str]], lengths: List[List[int]], device: torch.device) -> None:
        starts: Dict[str, int] = {}
        dims: Dict[str, int] = {}
        base = 0
        for ks, ls in zip(keys, lengths):
            off = 0
            for k, l in zip(ks, ls):
                if k not in starts:  # first occurrence wins, like KeyedTensor.regroup
                    starts[k], dims[k] = base + off, l
                off += l
            base += off
        idx: List[int] = []
        self._out_lengths = []
        for g in self._groups:
            n = 0
            for k in g:
                idx.extend(range(starts[k], starts[k] + dims[k]))
                n += dims[k]
            self._out_lengths.append(n)
        self._index = torch.tensor(idx, dtype=torch.long, device=device)

    def set_device(self, device: str) -> None:
        if self._index is not None:
            self._index = self._index.to(device)

    def forward(self, values: List[torch.Tensor]) -> List[torch.Tensor]:
        assert self._index is not None and self._out_lengths is not None, "call init_tensors first"
        cat = values[0] if len(values) == 1 else torch.cat(values, dim=1)
        return list(torch.index_select(cat, 1, self._index).split(self._out_lengths, dim=1))


def module_init(module: "KTRegroupAsDict", keyed_tensors: List[KeyedTensor]) -> None:
    """First-call setup of a ``KTRegroupAsDict``: check that the inputs agree on device and key dimension and build the cached
    permutation (``torchrec/modules/regroup.py:39-55``)."""
    assert len(keyed_tensors) > 0, "Empty list provided"
    assert all(kt.device() == keyed_tensors[0].device() for kt in keyed_tensors), "All inputs should be on the same device."
    assert all(kt.key_dim() == keyed_tensors[0].key_dim() for kt in keyed_tensors), "All inputs should have the same key_dim"
    assert keyed_tensors[0].key_dim() == 1, "regrouping needs key_dim 1"
    module._init_regroup(keyed_tensors)


class KTRegroupAsDict(nn.Module):
    """``forward(List[KeyedTensor]) -> {key_i: tensor of groups[i]}`` with the permutation cached after the first call."""

    def __init__(self, groups: List[List[str]], keys: List[str], emb_dtype: Optional[torch.dtype] = None) -> None:
        super().__init__()
        torch._C._log_api_usage_once(f"torchrec_b200.modules.{self.__class__.__name__}")
        assert len(groups) == len(keys), "Groups and keys should have same length"
        self._groups = groups
        self._keys = keys
        self._emb_dtype = emb_dtype
        self._is_inited = False
        self._permute_pooled_embs_impl = PermuteMultiEmbedding(groups)

    def _init_regroup(self, keyed_tensors: List[KeyedTensor]) -> None:
        self._permute_pooled_embs_impl.init_tensors([kt.keys() for kt in keyed_tensors], [kt.length_per_key() for kt in keyed_tensors], keyed_tensors[0].values().device)
        self._is_inited = True

    def forward(self, keyed_tensors: List[KeyedTensor]) -> Dict[str, torch.Tensor]:
        if not self._is_inited:
            module_init(self, keyed_tensors)
        values = [kt.values().to(self._emb_dtype) if self._emb_dtype is not None else kt.values() for kt in keyed_tensors]
        return dict(zip(self._keys, self._permute_pooled_embs_impl(values)))
