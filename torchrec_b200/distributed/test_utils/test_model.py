"""A small recommendation model and its synthetic input for sharding tests.

``ModelInput.generate`` draws one *global* batch and cuts it into ``world_size`` local batches, so that a sharded model fed the
local batches can be compared with an unsharded model fed the global one.  ``TestSparseNN`` is dense MLP + pooled embeddings
(unweighted and weighted tables) + an over arch; in training mode it returns ``(loss, prediction)``.
Counterpart of ``torchrec/distributed/test_utils/test_model.py:67-1960``."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple, Type, Union

import torch
from torch import nn

from torchrec_b200.distributed.embedding import EmbeddingCollectionSharder
from torchrec_b200.distributed.embedding_types import EmbeddingComputeKernel
from torchrec_b200.distributed.embeddingbag import EmbeddingBagCollectionSharder
from torchrec_b200.distributed.types import QuantizedCommCodecs
from torchrec_b200.modules.embedding_configs import BaseEmbeddingConfig, EmbeddingBagConfig, EmbeddingConfig
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection, EmbeddingCollection
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor, KeyedTensor
from torchrec_b200.streamable import Pipelineable


def _draw_kjt(tables: Sequence[BaseEmbeddingConfig], batch_size: int, pooling: Sequence[int], weighted: bool, gen: torch.Generator,
              indices_dtype: torch.dtype, lengths_dtype: torch.dtype, max_lengths: Optional[Sequence[int]] = None) -> Optional[KeyedJaggedTensor]:
    """Feature-major KJT with lengths ~ U[0, 2 * pooling] per bag (capped by ``max_lengths``)."""
    if not tables:
        return None
    keys: List[str] = []
    lengths: List[torch.Tensor] = []
    values: List[torch.Tensor] = []
    f = 0
    for t, avg in zip(tables, pooling):
        for name in t.feature_names:
            ln = torch.randint(0, 2 * avg + 1, (batch_size,), generator=gen)
            if max_lengths is not None:
                ln = ln.clamp(max=max_lengths[f])
            keys.append(name)
            lengths.append(ln)
            values.append(torch.randint(0, t.num_embeddings, (int(ln.sum()),), generator=gen))
            f += 1
    v = torch.cat(values).to(indices_dtype)
    w = torch.rand(v.numel(), generator=gen) if weighted else None
    return KeyedJaggedTensor(keys=keys, values=v, weights=w, lengths=torch.cat(lengths).to(lengths_dtype))


def _slice_batch(kjt: Optional[KeyedJaggedTensor], lo: int, hi: int, batch_size: int) -> Optional[KeyedJaggedTensor]:
    """Samples ``[lo, hi)`` of every feature of a feature-major KJT."""
    if kjt is None:
        return None
    F = len(kjt.keys())
    lengths = kjt.lengths().view(F, batch_size)
    offsets = torch.cat([lengths.new_zeros(1), lengths.reshape(-1).cumsum(0)])
    keep = torch.zeros(kjt.values().numel(), dtype=torch.bool)
    for f in range(F):
        keep[int(offsets[f * batch_size + lo]): int(offsets[f * batch_size + hi])] = True
    return KeyedJaggedTensor(keys=kjt.keys(), values=kjt.values()[keep], weights=kjt.weights()[keep] if kjt.weights_or_none() is not None else None,
                             lengths=lengths[:, lo:hi].reshape(-1).contiguous())


@dataclass
class ModelInput(Pipelineable):
    float_features: torch.Tensor
    idlist_features: Optional[KeyedJaggedTensor]
    idscore_features: Optional[KeyedJaggedTensor]
    label: torch.Tensor

    @staticmethod
    def generate(batch_size: int, world_size: int, num_float_features: int, tables: Sequence[BaseEmbeddingConfig],
                 weighted_tables: Optional[Sequence[BaseEmbeddingConfig]] = None, pooling_avg: int = 10,
                 tables_pooling: Optional[List[int]] = None, weighted_tables_pooling: Optional[List[int]] = None,
                 max_feature_lengths: Optional[List[int]] = None, device: Optional[torch.device] = None,
                 indices_dtype: torch.dtype = torch.int64, lengths_dtype: torch.dtype = torch.int64,
                 random_seed: Optional[int] = None) -> Tuple["ModelInput", List["ModelInput"]]:
        """``(global input of world_size * batch_size samples, [local input of batch_size samples per rank])``."""
        gen = torch.Generator()
        gen.manual_seed(random_seed if random_seed is not None else int(torch.randint(0, 2 ** 31, (1,))))
        weighted_tables = list(weighted_tables or [])
        total = batch_size * world_size
        idlist = _draw_kjt(tables, total, tables_pooling or [pooling_avg] * len(tables), False, gen, indices_dtype, lengths_dtype, max_feature_lengths)
        idscore = _draw_kjt(weighted_tables, total, weighted_tables_pooling or [pooling_avg] * len(weighted_tables), True, gen, indices_dtype, lengths_dtype)
        dense = torch.rand(total, num_float_features, generator=gen)
        label = torch.rand(total, generator=gen)
        whole = ModelInput(dense, idlist, idscore, label)
        parts = [ModelInput(dense[r * batch_size: (r + 1) * batch_size], _slice_batch(idlist, r * batch_size, (r + 1) * batch_size, total),
                            _slice_batch(idscore, r * batch_size, (r + 1) * batch_size, total), label[r * batch_size: (r + 1) * batch_size])
                 for r in range(world_size)]
        if device is not None:
            whole, parts = whole.to(device), [p.to(device) for p in parts]
        return whole, parts

    def to(self, device: torch.device, non_blocking: bool = False) -> "ModelInput":
        mv = lambda x: None if x is None else x.to(device=device, non_blocking=non_blocking)  # noqa: E731
        return ModelInput(mv(self.float_features), mv(self.idlist_features), mv(self.idscore_features), mv(self.label))

    def record_stream(self, stream: torch.Stream) -> None:
        for t in (self.float_features, self.label):
            if t.is_cuda:
                t.record_stream(stream)
        for k in (self.idlist_features, self.idscore_features):
            if k is not None:
                k.record_stream(stream)


class TestDenseArch(nn.Module):
    """``[B, num_float_features]`` -> ``[B, 8]``."""

    __test__ = False

    def __init__(self, num_float_features: int = 10, device: Optional[torch.device] = None) -> None:
        super().__init__()
        self.linear = nn.Linear(num_float_features, 8, device=device)

    def forward(self, dense_input: torch.Tensor) -> torch.Tensor:
        return self.linear(dense_input)


class TestOverArch(nn.Module):
    """Concatenates the dense vector with the chosen pooled embeddings and projects to 16 features."""

    __test__ = False

    def __init__(self, tables: Sequence[BaseEmbeddingConfig], weighted_tables: Sequence[BaseEmbeddingConfig],
                 embedding_names: Optional[List[str]] = None, device: Optional[torch.device] = None) -> None:
        super().__init__()
        self._features = embedding_names or [f for t in list(tables) + list(weighted_tables) for f in t.feature_names]
        dims = {f: t.embedding_dim for t in list(tables) + list(weighted_tables) for f in t.feature_names}
        in_features = 8 + sum(dims.get(f.split("@")[0], 0) for f in self._features)
        self.linear = nn.Linear(in_features, 16, device=device)

    def forward(self, dense: torch.Tensor, sparse: KeyedTensor) -> torch.Tensor:
        per_key = sparse.to_dict()
        return self.linear(torch.cat([dense] + [per_key[f] for f in self._features], dim=1))


class TestSparseArch(nn.Module):
    """Unweighted and weighted pooled collections side by side; the output carries the keys of both."""

    __test__ = False

    def __init__(self, tables: List[EmbeddingBagConfig], weighted_tables: List[EmbeddingBagConfig], device: Optional[torch.device] = None) -> None:
        super().__init__()
        self.ebc = EmbeddingBagCollection(tables=tables, device=device)
        self.weighted_ebc = EmbeddingBagCollection(tables=weighted_tables, is_weighted=True, device=device) if weighted_tables else None

    def forward(self, features: KeyedJaggedTensor, weighted_features: Optional[KeyedJaggedTensor] = None, batch_size: Optional[int] = None) -> KeyedTensor:
        out = self.ebc(features)
        if self.weighted_ebc is None or weighted_features is None:
            return out
        w = self.weighted_ebc(weighted_features)
        return KeyedTensor(keys=out.keys() + w.keys(), length_per_key=out.length_per_key() + w.length_per_key(), values=torch.cat([out.values(), w.values()], dim=1))


class TestECSparseArch(nn.Module):
    """Sequence embeddings summed per sample, returned as a KeyedTensor so the same over arch applies."""

    __test__ = False

    def __init__(self, tables: List[EmbeddingConfig], device: Optional[torch.device] = None) -> None:
        super().__init__()
        self.ec = EmbeddingCollection(tables=tables, device=device)
        self._dims = {f: t.embedding_dim for t in tables for f in t.feature_names}

    def forward(self, features: KeyedJaggedTensor, weighted_features: Optional[KeyedJaggedTensor] = None, batch_size: Optional[int] = None) -> KeyedTensor:
        out = self.ec(features)
        keys, cols = [], []
        for k, jt in out.items():
            B = jt.lengths().numel()
            seg = torch.repeat_interleave(torch.arange(B, device=jt.values().device), jt.lengths().long())
            cols.append(torch.zeros(B, jt.values().shape[1], dtype=jt.values().dtype, device=jt.values().device).index_add_(0, seg, jt.values()))
            keys.append(k)
        return KeyedTensor(keys=keys, length_per_key=[c.shape[1] for c in cols], values=torch.cat(cols, dim=1))


class TestSparseNNBase(nn.Module):
    __test__ = False

    def __init__(self, tables: Sequence[BaseEmbeddingConfig], weighted_tables: Optional[Sequence[BaseEmbeddingConfig]] = None,
                 embedding_groups: Optional[Dict[str, List[str]]] = None, dense_device: Optional[torch.device] = None,
                 sparse_device: Optional[torch.device] = None) -> None:
        super().__init__()
        self.tables, self.weighted_tables = list(tables), list(weighted_tables or [])
        self.embedding_groups = embedding_groups
        self.dense_device, self.sparse_device = dense_device, sparse_device


class TestSparseNN(TestSparseNNBase):
    """``forward(ModelInput)`` -> ``(loss, prediction)`` in training mode, ``prediction`` otherwise."""

    __test__ = False

    def __init__(self, tables: Union[List[EmbeddingBagConfig], List[EmbeddingConfig]], num_float_features: int = 10,
                 weighted_tables: Optional[List[EmbeddingBagConfig]] = None, embedding_groups: Optional[Dict[str, List[str]]] = None,
                 dense_device: Optional[torch.device] = None, sparse_device: Optional[torch.device] = None,
                 over_arch_clazz: Type[nn.Module] = TestOverArch, postproc_module: Optional[nn.Module] = None) -> None:
        super().__init__(tables, weighted_tables, embedding_groups, dense_device, sparse_device)
        weighted_tables = weighted_tables or []
        self.dense = TestDenseArch(num_float_features, dense_device)
        if isinstance(tables[0], EmbeddingConfig):
            self.sparse: nn.Module = TestECSparseArch(list(tables), sparse_device)
        else:
            self.sparse = TestSparseArch(list(tables), list(weighted_tables), sparse_device)
        names = list(embedding_groups.values())[0] if embedding_groups else None
        self.over = over_arch_clazz(tables, weighted_tables, names, dense_device)
        self.postproc_module = postproc_module

    def sparse_forward(self, input: ModelInput) -> KeyedTensor:
        return self.sparse(features=input.idlist_features, weighted_features=input.idscore_features, batch_size=input.float_features.size(0))

    def dense_forward(self, input: ModelInput, sparse_output: KeyedTensor):
        pred = torch.sigmoid(torch.mean(self.over(self.dense(input.float_features), sparse_output), dim=1))
        if self.training:
            return torch.nn.functional.binary_cross_entropy(pred, input.label), pred
        return pred

    def forward(self, input: ModelInput):
        if self.postproc_module is not None:
            input = self.postproc_module(input)
        return self.dense_forward(input, self.sparse_forward(input))


class _RestrictedSharderMixin:
    """Offer exactly one sharding type and one compute kernel to the planner."""

    def _restrict(self, sharding_type: str, kernel_type: str) -> None:
        self._sharding_type, self._kernel_type = sharding_type, kernel_type

    def sharding_types(self, compute_device_type: str) -> List[str]:
        return [self._sharding_type]

    def compute_kernels(self, sharding_type: str, compute_device_type: str) -> List[str]:
        return [self._kernel_type]


class TestEBCSharder(_RestrictedSharderMixin, EmbeddingBagCollectionSharder):
    __test__ = False

    def __init__(self, sharding_type: str, kernel_type: str = EmbeddingComputeKernel.FUSED.value, fused_params: Optional[Dict[str, Any]] = None,
                 qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None) -> None:
        EmbeddingBagCollectionSharder.__init__(self, fused_params if fused_params is not None else {"learning_rate": 0.1}, qcomm_codecs_registry)
        self._restrict(sharding_type, kernel_type)


class TestECSharder(_RestrictedSharderMixin, EmbeddingCollectionSharder):
    __test__ = False

    def __init__(self, sharding_type: str, kernel_type: str = EmbeddingComputeKernel.FUSED.value, fused_params: Optional[Dict[str, Any]] = None,
                 qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None, use_index_dedup: bool = False) -> None:
        EmbeddingCollectionSharder.__init__(self, fused_params if fused_params is not None else {"learning_rate": 0.1}, qcomm_codecs_registry, use_index_dedup=use_index_dedup)
        self._restrict(sharding_type, kernel_type)
