"""Grouped lookups of sharded inference: one process drives every device, so a lookup holds the quantized kernels of ALL ranks.

``MetaInferGrouped(Pooled)EmbeddingsLookup`` is what one device holds (a list of quantized kernels, one per group of tables);
``InferGrouped(Pooled)EmbeddingsLookup`` is the per-rank list of those and maps the input distribution's per-device features to
per-device outputs.  Counterpart of ``torchrec/distributed/embedding_lookup.py:820-1340``."""
from __future__ import annotations

from collections import OrderedDict
from typing import Any, Dict, Iterator, List, Optional, Tuple, Type, Union

import torch
from torch import nn

from torchrec_b200.distributed.embedding_types import BaseEmbeddingLookup, GroupedEmbeddingConfig, InputDistOutputs
from torchrec_b200.distributed.fused_params import TBEToRegisterMixIn, get_tbes_to_register_from_iterable
from torchrec_b200.distributed.quant_embedding_kernel import QuantBatchedEmbedding, QuantBatchedEmbeddingBag
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


def _device_of_rank(device_type: str, rank: int) -> torch.device:
    return torch.device(device_type, rank) if device_type == "cuda" else torch.device(device_type)


class _DeviceLookup(nn.Module, TBEToRegisterMixIn):
    """The kernels one device holds; ``_kernel`` and ``_cat_dim`` distinguish the pooled from the sequence form."""

    _kernel: Type[nn.Module] = QuantBatchedEmbeddingBag
    _cat_dim = 1  # pooled groups sit side by side; rows of sequence groups follow one another

    def __init__(self, grouped_configs: List[GroupedEmbeddingConfig], device: Optional[torch.device] = None,
                 feature_processor: Optional[nn.Module] = None, fused_params: Optional[Dict[str, Any]] = None, shard_index: Optional[int] = None) -> None:
        super().__init__()
        self.grouped_configs = grouped_configs
        self._feature_splits = [c.num_features() for c in grouped_configs]
        self._emb_modules = nn.ModuleList([self._kernel(c, device=device, fused_params=fused_params) for c in grouped_configs])
        self._feature_processor = feature_processor
        self._device = device
        wanted = (fused_params or {}).get("output_dtype")
        self.output_dtype: torch.dtype = wanted if isinstance(wanted, torch.dtype) else torch.float32

    def get_tbes_to_register(self) -> Dict[nn.Module, GroupedEmbeddingConfig]:
        return get_tbes_to_register_from_iterable(self._emb_modules)

    def forward(self, sparse_features: KeyedJaggedTensor) -> torch.Tensor:
        if not self.grouped_configs:
            return torch.empty([0], dtype=self.output_dtype, device=self._device if self._device is not None and self._device.type != "meta" else None)
        parts = [sparse_features] if len(self._feature_splits) == 1 else sparse_features.split(self._feature_splits)
        if self._feature_processor is not None:
            parts = [self._feature_processor(p) if c.has_feature_processor else p for c, p in zip(self.grouped_configs, parts)]
        outs = [kernel(p) for kernel, p in zip(self._emb_modules, parts)]
        return outs[0] if len(outs) == 1 else torch.cat(outs, dim=self._cat_dim)

    # the state is the kernels' packed tables, under ``<table>.weight``
    def state_dict(self, destination: Optional[Dict[str, Any]] = None, prefix: str = "", keep_vars: bool = False) -> Dict[str, Any]:
        out = OrderedDict() if destination is None else destination
        for name, buf in self.named_buffers(prefix.rstrip(".")):
            out[name] = buf
        return out

    def load_state_dict(self, state_dict: Dict[str, torch.Tensor], strict: bool = True):  # type: ignore[override]
        from torch.nn.modules.module import _IncompatibleKeys

        mine = dict(self.named_buffers())
        missing = [k for k in mine if k not in state_dict]
        unexpected = [k for k in state_dict if k not in mine]
        for k, dst in mine.items():
            if k in state_dict:
                dst.copy_(state_dict[k].view(dst.dtype).reshape(dst.shape) if state_dict[k].dtype != dst.dtype else state_dict[k].reshape(dst.shape))
        if strict and (missing or unexpected):
            raise RuntimeError(f"missing keys {missing}, unexpected keys {unexpected}")
        return _IncompatibleKeys(missing_keys=missing, unexpected_keys=unexpected)

    def named_parameters(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True) -> Iterator[Tuple[str, nn.Parameter]]:
        yield from ()

    def named_buffers(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True) -> Iterator[Tuple[str, torch.Tensor]]:
        for kernel in self._emb_modules:
            yield from kernel.named_buffers(prefix, recurse)

    def flush(self) -> None:  # nothing is cached outside the tables
        pass

    def purge(self) -> None:
        pass


class MetaInferGroupedPooledEmbeddingsLookup(_DeviceLookup, BaseEmbeddingLookup[KeyedJaggedTensor, torch.Tensor]):
    _kernel, _cat_dim = QuantBatchedEmbeddingBag, 1


class MetaInferGroupedEmbeddingsLookup(_DeviceLookup, BaseEmbeddingLookup[KeyedJaggedTensor, torch.Tensor]):
    _kernel, _cat_dim = QuantBatchedEmbedding, 0


class _AllDevicesLookup(nn.Module, TBEToRegisterMixIn):
    """One ``_DeviceLookup`` per rank that holds tables; ``forward`` takes the input distribution's per-rank features."""

    _per_device: Type[_DeviceLookup] = MetaInferGroupedPooledEmbeddingsLookup

    def __init__(self, grouped_configs_per_rank: List[List[GroupedEmbeddingConfig]], world_size: int, fused_params: Optional[Dict[str, Any]] = None,
                 device: Optional[torch.device] = None, device_type_from_sharding_infos: Optional[Union[str, Tuple[str, ...]]] = None) -> None:
        super().__init__()
        kind = "meta" if device is not None and device.type == "meta" else ("cpu" if device is not None and device.type == "cpu" else "cuda")
        mixed = isinstance(device_type_from_sharding_infos, tuple)  # one table over several device types: the shard index names the rank
        self._is_empty_rank = [len(grouped_configs_per_rank[r]) == 0 for r in range(world_size)]
        self._embedding_lookups_per_rank = nn.ModuleList([
            self._per_device(grouped_configs_per_rank[r], device=_device_of_rank(kind, r), fused_params=fused_params, shard_index=r if mixed else None)
            for r in range(world_size) if not self._is_empty_rank[r]])

    def get_tbes_to_register(self) -> Dict[nn.Module, GroupedEmbeddingConfig]:
        return get_tbes_to_register_from_iterable(self._embedding_lookups_per_rank)

    def forward(self, input_dist_outputs: InputDistOutputs) -> List[torch.Tensor]:
        features = [f for f, empty in zip(input_dist_outputs.features, self._is_empty_rank) if not empty]
        return [lookup(f) for lookup, f in zip(self._embedding_lookups_per_rank, features)]

    def state_dict(self, destination: Optional[Dict[str, Any]] = None, prefix: str = "", keep_vars: bool = False) -> Dict[str, Any]:
        out = OrderedDict() if destination is None else destination
        for lookup in self._embedding_lookups_per_rank:
            lookup.state_dict(out, prefix, keep_vars)
        return out

    def named_parameters(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True) -> Iterator[Tuple[str, nn.Parameter]]:
        yield from ()

    def named_buffers(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True) -> Iterator[Tuple[str, torch.Tensor]]:
        for lookup in self._embedding_lookups_per_rank:
            yield from lookup.named_buffers(prefix, recurse)


class InferGroupedPooledEmbeddingsLookup(_AllDevicesLookup, BaseEmbeddingLookup[InputDistOutputs, List[torch.Tensor]]):
    _per_device = MetaInferGroupedPooledEmbeddingsLookup


class InferGroupedEmbeddingsLookup(_AllDevicesLookup, BaseEmbeddingLookup[InputDistOutputs, List[torch.Tensor]]):
    _per_device = MetaInferGroupedEmbeddingsLookup


class InferCPUGroupedEmbeddingsLookup(InferGroupedEmbeddingsLookup):
    """The sequence lookup with every rank's tables on the host."""

    def __init__(self, grouped_configs_per_rank: List[List[GroupedEmbeddingConfig]], world_size: int, fused_params: Optional[Dict[str, Any]] = None,
                 device: Optional[torch.device] = None) -> None:
        super().__init__(grouped_configs_per_rank, world_size, fused_params, torch.device("cpu"))
