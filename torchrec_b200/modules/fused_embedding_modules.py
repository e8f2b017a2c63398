"""Single-device embedding collections backed by the table-batched kernel with the optimizer fused into backward.

``FusedEmbeddingBagCollection(tables, optimizer_type, optimizer_kwargs)`` behaves like ``EmbeddingBagCollection`` but all
tables live in one ``TableBatchedEmbeddingBags`` per (pooling, dim-compatible) group and are updated inside the backward
kernel; ``fuse_embedding_optimizer`` swaps the plain modules of a model for these.  Counterpart of
``torchrec/modules/fused_embedding_modules.py:281,529,793``.
"""
from __future__ import annotations

import copy
from collections import defaultdict
from typing import Any, Dict, Iterator, List, Optional, Tuple, Type

import torch
from torch import nn

from torchrec_b200.distributed.utils import optimizer_type_to_emb_opt_type
from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig, EmbeddingConfig, PoolingMode, PoolingType, data_type_to_dtype, pooling_type_to_pooling_mode
from torchrec_b200.modules.embedding_modules import (
    EmbeddingBagCollection, EmbeddingBagCollectionInterface, EmbeddingCollection, EmbeddingCollectionInterface, get_embedding_names_by_table,
)
from torchrec_b200.ops.tbe import EmbOptimType, OptimizerArgs, TableBatchedEmbeddingBags
from torchrec_b200.optim.fused import FusedOptimizer, FusedOptimizerModule
from torchrec_b200.optim.keyed import CombinedOptimizer, KeyedOptimizer
from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor, KeyedTensor


def _optimizer_args(optimizer_type: Type[torch.optim.Optimizer], kwargs: Dict[str, Any]) -> OptimizerArgs:
    k = dict(kwargs)
    return OptimizerArgs(optimizer=optimizer_type_to_emb_opt_type(optimizer_type), learning_rate=float(k.get("lr", k.get("learning_rate", 0.01))),
                         eps=float(k.get("eps", 1e-8)), beta1=float(k.get("betas", (0.9, 0.999))[0]) if "betas" in k else float(k.get("beta1", 0.9)),
                         beta2=float(k.get("betas", (0.9, 0.999))[1]) if "betas" in k else float(k.get("beta2", 0.999)),
                         weight_decay=float(k.get("weight_decay", 0.0)), eta=float(k.get("eta", 0.001)))


class _TbeFusedOptimizer(FusedOptimizer):
    """Keyed view of the kernel-side optimizer: params are the table views, state the per-table state views."""

    def __init__(self, emb: TableBatchedEmbeddingBags, table_names: List[str], prefix: str) -> None:
        self._emb = emb
        params: Dict[str, torch.Tensor] = {}
        state: Dict[Any, Any] = {}
        group = {"params": [], "lr": emb.optimizer_args.learning_rate}
        for name, w, st in zip(table_names, emb.split_embedding_weights(), emb.split_optimizer_states()):
            params[f"{prefix}{name}.weight"] = w
            group["params"].append(w)
            state[w] = {f"{name}.{k}": v for k, v in st.items()}
        super().__init__(params, state, [group])

    def zero_grad(self, set_to_none: bool = False) -> None:
        pass

    def step(self, closure: Any = None) -> None:
        for g in self.param_groups:
            self._emb.set_learning_rate(g["lr"])


EmbeddingFusedOptimizer = _TbeFusedOptimizer  # the reference's name for the keyed view of a kernel-side optimizer


def convert_optimizer_type_and_kwargs(optimizer_type: Type[torch.optim.Optimizer], optimizer_kwargs: Dict[str, Any]):
    """``(kernel optimizer, kernel arguments)`` for an optimizer class of torch or of this package (``lr`` becomes
    ``learning_rate``), or ``None`` when the embedding kernels have no fused form of it."""
    try:
        kind = optimizer_type_to_emb_opt_type(optimizer_type)
    except Exception:
        return None
    if kind is None:
        return None
    kwargs = dict(optimizer_kwargs)
    if "lr" in kwargs:
        kwargs["learning_rate"] = kwargs.pop("lr")
    return kind, kwargs


class _FusedBase(FusedOptimizerModule):
    _container = "embedding_bags"

    def _build(self, tables, optimizer_type, optimizer_kwargs, device, pooled: bool, is_weighted: bool = False) -> None:
        self._optimizer_type = optimizer_type
        self._optimizer_kwargs = optimizer_kwargs
        self._device = device if device is not None else torch.device("cpu")
        groups: Dict[Any, List[Any]] = defaultdict(list)
        for t in tables:
            groups[(t.pooling if pooled else PoolingType.NONE, t.data_type)].append(t)
        self._emb_modules = nn.ModuleList()
        self._group_tables: List[List[Any]] = []
        self._feature_splits: List[int] = []
        container = nn.ModuleDict()
        setattr(self, self._container, container)
        optims: List[Tuple[str, KeyedOptimizer]] = []
        for (pooling, data_type), group in groups.items():
            mode = pooling_type_to_pooling_mode(pooling) if pooled else PoolingMode.NONE
            emb = TableBatchedEmbeddingBags([(t.num_embeddings, t.embedding_dim) for t in group], [i for i, t in enumerate(group) for _ in t.feature_names], mode,
                                            data_type_to_dtype(data_type), torch.float32, _optimizer_args(optimizer_type, optimizer_kwargs), fused=True,
                                            device=self._device if self._device.type != "meta" else None)
            for t, w in zip(group, emb.split_embedding_weights()):
                if self._device.type != "meta":
                    with torch.no_grad():
                        if t.init_fn is not None:
                            t.init_fn(w)
                        else:
                            w.uniform_(t.get_weight_init_min(), t.get_weight_init_max())
                holder = nn.Module()
                p = nn.Parameter(w, requires_grad=False)
                p._in_backward_optimizers = [None]  # updated by the kernel: dense optimizers must skip it
                holder.register_parameter("weight", p)
                container[t.name] = holder
            self._emb_modules.append(emb)
            self._group_tables.append(group)
            self._feature_splits.append(sum(len(t.feature_names) for t in group))
            optims.append(("", _TbeFusedOptimizer(emb, [t.name for t in group], f"{self._container}.")))
        self._optim = CombinedOptimizer(optims)
        self._feature_names = [f for g in self._group_tables for t in g for f in t.feature_names]

    @property
    def fused_optimizer(self) -> KeyedOptimizer:
        return self._optim

    def _lookup(self, features: KeyedJaggedTensor, weighted: bool) -> List[Tuple[KeyedJaggedTensor, torch.Tensor, List[Any]]]:
        kjt = features.permute([features.keys().index(f) for f in self._feature_names]) if features.keys() != self._feature_names else features
        parts = kjt.split(self._feature_splits) if len(self._emb_modules) > 1 else [kjt]
        out = []
        for emb, f, group in zip(self._emb_modules, parts, self._group_tables):
            out.append((f, emb(f.values(), f.offsets(), f.weights_or_none() if weighted else None, batch_size=f.stride()), group))
        return out


class FusedEmbeddingBagCollection(EmbeddingBagCollectionInterface, _FusedBase):
    _container = "embedding_bags"

    def __init__(self, tables: List[EmbeddingBagConfig], optimizer_type: Type[torch.optim.Optimizer], optimizer_kwargs: Dict[str, Any], is_weighted: bool = False,
                 device: Optional[torch.device] = None, location=None) -> None:
        super().__init__()
        self._is_weighted = is_weighted
        self._embedding_bag_configs = tables
        self._build(tables, optimizer_type, optimizer_kwargs, device, pooled=True, is_weighted=is_weighted)
        self._embedding_names = [n for names in get_embedding_names_by_table(tables) for n in names]
        name_of = dict(zip([f"{t.name}:{f}" for t in tables for f in t.feature_names], self._embedding_names))
        grouped = [name_of[f"{t.name}:{f}"] for g in self._group_tables for t in g for f in t.feature_names]
        self._grouped_dims = [t.embedding_dim for g in self._group_tables for t in g for _ in t.feature_names]
        self._out_perm = None if grouped == self._embedding_names else [grouped.index(n) for n in self._embedding_names]
        self._length_per_key = [t.embedding_dim for t in tables for _ in t.feature_names]

    def forward(self, features: KeyedJaggedTensor) -> KeyedTensor:
        outs = [o for _, o, _ in self._lookup(features, self._is_weighted)]
        values = outs[0] if len(outs) == 1 else torch.cat(outs, dim=1)
        if self._out_perm is not None:
            pieces = values.split(self._grouped_dims, dim=1)
            values = torch.cat([pieces[i] for i in self._out_perm], dim=1)
        return KeyedTensor(keys=self._embedding_names, values=values, length_per_key=self._length_per_key)

    def embedding_bag_configs(self) -> List[EmbeddingBagConfig]:
        return self._embedding_bag_configs

    def is_weighted(self) -> bool:
        return self._is_weighted


class FusedEmbeddingCollection(EmbeddingCollectionInterface, _FusedBase):
    _container = "embeddings"

    def __init__(self, tables: List[EmbeddingConfig], optimizer_type: Type[torch.optim.Optimizer], optimizer_kwargs: Dict[str, Any],
                 device: Optional[torch.device] = None, need_indices: bool = False, location=None) -> None:
        super().__init__()
        self._embedding_configs = tables
        self._need_indices = need_indices
        self._embedding_dim = tables[0].embedding_dim if tables else -1
        self._build(tables, optimizer_type, optimizer_kwargs, device, pooled=False)
        self._embedding_names_by_table = get_embedding_names_by_table(tables)
        self._name_of = {f"{t.name}:{f}": n for t, names in zip(tables, self._embedding_names_by_table) for f, n in zip(t.feature_names, names)}

    def forward(self, features: KeyedJaggedTensor) -> Dict[str, JaggedTensor]:
        out: Dict[str, JaggedTensor] = {}
        for f, rows, group in self._lookup(features, False):
            lpk = f.length_per_key()
            pieces = rows.split(lpk, dim=0)
            lengths = f.lengths().view(-1, f.stride())
            vals = f.values().split(lpk) if self._need_indices else None
            i = 0
            for t in group:
                for feat in t.feature_names:
                    out[self._name_of[f"{t.name}:{feat}"]] = JaggedTensor(values=pieces[i], lengths=lengths[i], weights=vals[i] if vals is not None else None)
                    i += 1
        return out

    def embedding_configs(self) -> List[EmbeddingConfig]:
        return self._embedding_configs

    def embedding_dim(self) -> int:
        return self._embedding_dim

    def embedding_names_by_table(self) -> List[List[str]]:
        return self._embedding_names_by_table

    def need_indices(self) -> bool:
        return self._need_indices


def fuse_embedding_optimizer(model: nn.Module, optimizer_type: Type[torch.optim.Optimizer], optimizer_kwargs: Dict[str, Any], device: torch.device, location=None) -> nn.Module:
    """Replace every ``EmbeddingBagCollection`` / ``EmbeddingCollection`` under ``model`` by its fused counterpart (weights copied)."""

    def convert(m: nn.Module) -> Optional[nn.Module]:
        if type(m) is EmbeddingBagCollection:
            new = FusedEmbeddingBagCollection(copy.deepcopy(m.embedding_bag_configs()), optimizer_type, optimizer_kwargs, m.is_weighted(), device)
            src = m.embedding_bags
        elif type(m) is EmbeddingCollection:
            new = FusedEmbeddingCollection(copy.deepcopy(m.embedding_configs()), optimizer_type, optimizer_kwargs, device, m.need_indices())
            src = m.embeddings
        else:
            return None
        with torch.no_grad():
            for name, holder in getattr(new, new._container).items():
                if src[name].weight.device.type != "meta":
                    holder.weight.copy_(src[name].weight.to(holder.weight.device))
        return new

    root = convert(model)
    if root is not None:
        return root
    for parent in list(model.modules()):
        for name, child in list(parent.named_children()):
            new = convert(child)
            if new is not None:
                setattr(parent, name, new)
    return model
