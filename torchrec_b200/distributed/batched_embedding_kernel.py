"""Per-rank embedding kernels: a group of table shards backed by one ``TableBatchedEmbeddingBags``.

``BatchedFusedEmbeddingBag`` / ``BatchedFusedEmbedding`` (pooled / unpooled, optimizer fused into
backward) and ``BatchedDenseEmbeddingBag`` / ``BatchedDenseEmbedding`` (dense gradient, for
data-parallel tables).  ``EmbeddingFusedOptimizer`` exposes the fused optimizer state as
``ShardedTensor``s named ``<table>.momentum1`` / ``<table>.momentum2`` so that it is checkpointed
like any keyed optimizer; row-wise states are sharded along rows even for column-wise tables.

Counterpart of ``torchrec/distributed/batched_embedding_kernel.py`` (optimizer ``:1068-1489``,
per-table views ``:1492-1590``, kernels ``:2302-3350``) and ``embedding_kernel.py:221-379``.
"""
from __future__ import annotations

import copy
import itertools
from typing import Any, Dict, Iterator, List, Optional, Tuple, Union

import torch
import torch.distributed as dist
from torch import nn
from torch.distributed._shard.sharded_tensor import Shard, ShardedTensor, ShardedTensorMetadata, TensorProperties
from torch.distributed._shard.sharding_spec import ShardMetadata

from torchrec_b200.distributed.embedding_types import BaseEmbeddingLookup, GroupedEmbeddingConfig, ShardedEmbeddingTable
from torchrec_b200.distributed.types import ShardingType
from torchrec_b200.modules.embedding_configs import (
    PoolingMode,
    PoolingType,
    data_type_to_dtype,
    pooling_type_to_pooling_mode,
)
from torchrec_b200.ops.tbe import EmbOptimType, OptimizerArgs, TableBatchedEmbeddingBags, TBEPlan
from torchrec_b200.optim.fused import FusedOptimizer, FusedOptimizerModule
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class TableBatchedEmbeddingSlice(nn.Parameter):
    """A parameter that is a ``[rows, cols]`` view of one table inside the flat TBE buffer."""

    __slots__ = ["_original_tensor", "_start_offset", "_end_offset", "_num_embeddings", "_embedding_dim"]

    def __new__(cls, data: torch.Tensor, start_offset: int, end_offset: int, num_embeddings: int, embedding_dim: int):
        view = data.detach()[start_offset:end_offset].view(num_embeddings, embedding_dim)
        obj = torch.Tensor._make_subclass(cls, view, data.requires_grad)
        obj._original_tensor = data
        obj._start_offset, obj._end_offset = start_offset, end_offset
        obj._num_embeddings, obj._embedding_dim = num_embeddings, embedding_dim
        return obj

    def __deepcopy__(self, memo):
        new_original = copy.deepcopy(self._original_tensor, memo)
        return TableBatchedEmbeddingSlice(new_original, self._start_offset, self._end_offset, self._num_embeddings, self._embedding_dim)

    @property
    def grad(self):
        g = self._original_tensor.grad
        if g is None:
            return None
        return g[self._start_offset: self._end_offset].view(self._num_embeddings, self._embedding_dim)

    @grad.setter
    def grad(self, set_grad):
        if set_grad is None:
            self._original_tensor.grad = None
        elif self._original_tensor.grad is not None:
            self._original_tensor.grad[self._start_offset: self._end_offset].copy_(set_grad.view(-1))

    @property
    def grad_fn(self):
        return None


def _optimizer_args_from_fused_params(fused_params: Optional[Dict[str, Any]]) -> OptimizerArgs:
    fp = fused_params or {}
    opt = fp.get("optimizer", EmbOptimType.EXACT_SGD)
    if isinstance(opt, str):
        opt = EmbOptimType(opt)
    betas = fp.get("betas", None)
    return OptimizerArgs(
        optimizer=opt,
        learning_rate=float(fp.get("learning_rate", fp.get("lr", 0.01))),
        eps=float(fp.get("eps", 1.0e-8)),
        beta1=float(fp.get("beta1", betas[0] if betas else 0.9)),
        beta2=float(fp.get("beta2", betas[1] if betas else 0.999)),
        weight_decay=float(fp.get("weight_decay", 0.0)),
        eta=float(fp.get("eta", 0.001)),
        max_gradient=float(fp.get("max_gradient", 1.0)) if fp.get("gradient_clipping", False) else 0.0,
        stochastic_rounding=bool(fp.get("stochastic_rounding", True)),
    )


_ROWWISE_STATE = {
    EmbOptimType.EXACT_ROWWISE_ADAGRAD: {"momentum1"},
    EmbOptimType.PARTIAL_ROWWISE_ADAM: {"momentum2"},
    EmbOptimType.PARTIAL_ROWWISE_LAMB: {"momentum2"},
}


class EmbeddingFusedOptimizer(FusedOptimizer):
    """View of the optimizer state that lives inside a TBE, keyed by ``<table>.weight``.

    The state of table ``t`` is ``{"<t>.momentum1": ShardedTensor, ...}`` whose local shard is a
    view into the TBE state buffer, so checkpoint loads write straight into the kernel's memory.
    ``step`` only publishes a changed learning rate to the kernel.
    """

    def __init__(self, config: GroupedEmbeddingConfig, emb_module: TableBatchedEmbeddingBags, pg: Optional[dist.ProcessGroup] = None,
                 create_for_table: Optional[str] = None, param_weight_for_table: Optional[nn.Parameter] = None,
                 embedding_weights_by_table: Optional[List[torch.Tensor]] = None, all_optimizer_states: Optional[List[Dict[str, torch.Tensor]]] = None) -> None:
        self._emb_module = emb_module
        self._pg = pg
        params: Dict[str, Union[torch.Tensor, ShardedTensor]] = {}
        state: Dict[Any, Any] = {}
        param_group: Dict[str, Any] = {"params": [], "lr": emb_module.optimizer_args.learning_rate}
        weights = embedding_weights_by_table if embedding_weights_by_table is not None else emb_module.split_embedding_weights()
        states = all_optimizer_states if all_optimizer_states is not None else emb_module.split_optimizer_states()
        rowwise_names = _ROWWISE_STATE.get(emb_module.optimizer_args.optimizer, set())
        world = dist.get_world_size(pg) if pg is not None else 1
        rank = dist.get_rank(pg) if pg is not None else 0
        # group shards of the same table (column-wise puts several shards of one table on a rank)
        by_name: Dict[str, List[int]] = {}
        for i, t in enumerate(config.embedding_tables):
            by_name.setdefault(t.name, []).append(i)
        for name, idxs in by_name.items():
            if create_for_table is not None and create_for_table != name:
                continue
            tables = [config.embedding_tables[i] for i in idxs]
            t0 = tables[0]
            weight = param_weight_for_table if param_weight_for_table is not None else weights[idxs[0]]
            key = f"{name}.weight"
            params[key] = weight
            param_group["params"].append(weight)
            st: Dict[str, Any] = {}
            for sname in states[idxs[0]].keys():
                local = [states[i][sname] for i in idxs]
                st[f"{name}.{sname}"] = self._wrap_state(t0, tables, local, sname in rowwise_names, world, rank)
            state[weight] = st
        super().__init__(params, state, [param_group])

    def _wrap_state(self, t0: ShardedEmbeddingTable, tables: List[ShardedEmbeddingTable], local: List[torch.Tensor], rowwise: bool, world: int, rank: int):
        gm = t0.global_metadata
        if gm is None or self._pg is None:
            return local[0] if len(local) == 1 else torch.cat([x.reshape(x.shape[0], -1) for x in local], dim=-1)
        local_shards: List[Shard] = []
        if rowwise:
            # one value per row of every shard.  Column shards of the same rows keep independent values (each is computed from
            # its own columns), so the state tensor stacks the shards along dim 0 in (column offset, row offset) order:
            # row-wise tables give [rows], column-wise ones [rows * column shards]
            # (same layout as torchrec/distributed/batched_embedding_kernel.py:1132-1190).
            ordered = sorted(gm.shards_metadata, key=lambda sm: (sm.shard_offsets[1], sm.shard_offsets[0], str(sm.placement)))
            offset_of: Dict[Tuple[Any, ...], int] = {}
            metas = []
            rolling = 0
            for sm in ordered:
                k = (sm.shard_offsets[0], sm.shard_offsets[1], sm.shard_sizes[0], sm.shard_sizes[1], str(sm.placement))
                offset_of[k] = rolling
                metas.append(ShardMetadata(shard_offsets=[rolling], shard_sizes=[sm.shard_sizes[0]], placement=copy.deepcopy(sm.placement)))
                rolling += sm.shard_sizes[0]
            for t, x in zip(tables, local):
                lm = t.local_metadata
                k = (lm.shard_offsets[0], lm.shard_offsets[1], lm.shard_sizes[0], lm.shard_sizes[1], str(lm.placement))
                local_shards.append(Shard(x, ShardMetadata(shard_offsets=[offset_of[k]], shard_sizes=[lm.shard_sizes[0]], placement=copy.deepcopy(lm.placement))))
            size = torch.Size([rolling])
        else:
            metas = [copy.deepcopy(sm) for sm in gm.shards_metadata]
            for t, x in zip(tables, local):
                local_shards.append(Shard(x, copy.deepcopy(t.local_metadata)))
            size = gm.size
        meta = ShardedTensorMetadata(
            shards_metadata=metas, size=size,
            tensor_properties=TensorProperties(dtype=local[0].dtype, layout=local[0].layout, requires_grad=False),
        )
        return ShardedTensor._init_from_local_shards_and_global_metadata(local_shards=local_shards, sharded_tensor_metadata=meta, process_group=self._pg)

    def zero_grad(self, set_to_none: bool = False) -> None:
        pass

    def step(self, closure: Any = None) -> None:
        # the update already happened in backward; only hyper-parameters flow from param_groups to the kernel
        for group in self.param_groups:
            if "lr" in group:
                self._emb_module.set_learning_rate(group["lr"])

    def set_optimizer_step(self, step: int) -> None:
        self._emb_module.step = int(step)

    def update_hyper_parameters(self, params_dict: Dict[str, Any]) -> None:
        for k, v in params_dict.items():
            if k in ("lr", "learning_rate"):
                self._emb_module.set_learning_rate(v)
                for g in self.param_groups:
                    g["lr"] = v
            elif hasattr(self._emb_module.optimizer_args, k):
                setattr(self._emb_module.optimizer_args, k, v)


class BaseEmbedding(BaseEmbeddingLookup[KeyedJaggedTensor, torch.Tensor]):
    """Common part of the four kernels below."""

    def __init__(self, config: GroupedEmbeddingConfig, pg: Optional[dist.ProcessGroup], device: Optional[torch.device],
                 pooling_mode: PoolingMode, fused: bool, sharding_type: Optional[ShardingType] = None) -> None:
        super().__init__()
        self._config = config
        self._pg = pg
        self._sharding_type = sharding_type
        self._local_rows = [t.local_rows for t in config.embedding_tables]
        self._local_cols = [t.local_cols for t in config.embedding_tables]
        self._feature_table_map: List[int] = []
        self._num_embeddings = [t.num_embeddings for t in config.embedding_tables]
        for idx, t in enumerate(config.embedding_tables):
            self._feature_table_map.extend([idx] * t.num_features())
        fp = config.fused_params or {}
        out_dtype = fp.get("output_dtype", None)
        if out_dtype is not None and not isinstance(out_dtype, torch.dtype):
            out_dtype = data_type_to_dtype(out_dtype)
        self._emb_module = TableBatchedEmbeddingBags(
            embedding_specs=list(zip(self._local_rows, self._local_cols)),
            feature_table_map=self._feature_table_map,
            pooling_mode=pooling_mode,
            weights_precision=data_type_to_dtype(config.data_type),
            output_dtype=out_dtype or torch.float32,
            optimizer_args=_optimizer_args_from_fused_params(config.fused_params),
            fused=fused,
            device=device,
        )
        self._fused = fused
        self.init_parameters()

    @property
    def emb_module(self) -> TableBatchedEmbeddingBags:
        return self._emb_module

    @property
    def config(self) -> GroupedEmbeddingConfig:
        return self._config

    def init_parameters(self) -> None:
        if self._emb_module.weights.device.type == "meta":
            return
        for (rows, dim, table), param in zip(
            zip(self._local_rows, self._local_cols, self._config.embedding_tables), self._emb_module.split_embedding_weights()
        ):
            if rows == 0:
                continue
            assert table.init_fn is not None
            if param.dtype == torch.float32:
                table.init_fn(param)
            else:
                tmp = torch.empty(param.shape, dtype=torch.float32, device=param.device)
                table.init_fn(tmp)
                param.copy_(tmp)

    def forward(self, features: KeyedJaggedTensor, plan: Optional[TBEPlan] = None) -> torch.Tensor:
        weights = features.weights_or_none()
        if weights is not None and not torch.is_floating_point(weights):
            weights = None
        if not self._config.is_weighted:
            weights = None
        return self._emb_module(
            indices=features.values(), offsets=features.offsets(), per_sample_weights=weights,
            batch_size=features.stride() if not features.variable_stride_per_key() else None, plan=plan,
        )

    def build_plan(self, features: KeyedJaggedTensor) -> Optional[TBEPlan]:
        weights = features.weights_or_none() if self._config.is_weighted else None
        return self._emb_module.build_plan(features.values(), features.offsets(), weights, features.stride())

    def split_embedding_weights(self) -> List[torch.Tensor]:
        return self._emb_module.split_embedding_weights()

    def named_split_embedding_weights(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True) -> Iterator[Tuple[str, torch.Tensor]]:
        for config, tensor in zip(self._config.embedding_tables, self.split_embedding_weights()):
            key = f"{prefix}.{config.name}.weight" if prefix else f"{config.name}.weight"
            yield key, tensor

    def named_buffers(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True):
        # weights of fused kernels are reported as buffers: no autograd gradient, no dense optimizer
        if self._fused:
            yield from self.named_split_embedding_weights(prefix)
        else:
            yield from ()

    def named_parameters(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True):
        if self._fused or not recurse:
            # recurse=False is how DDP enumerates: the flat buffer is reported by the TBE module itself
            yield from ()
            return
        w = self._emb_module.weights
        offs = self._emb_module.weights_offsets
        for i, t in enumerate(self._config.embedding_tables):
            key = f"{prefix}.{t.name}.weight" if prefix else f"{t.name}.weight"
            yield key, TableBatchedEmbeddingSlice(w, offs[i], offs[i + 1], self._local_rows[i], self._local_cols[i])

    def parameters(self, recurse: bool = True):
        for _, p in self.named_parameters():
            yield p

    def flush(self) -> None:
        pass

    def purge(self) -> None:
        pass

    def state_dict(self, destination=None, prefix: str = "", keep_vars: bool = False):
        if destination is None:
            destination = {}
        for k, v in self.named_split_embedding_weights(prefix.rstrip(".")):
            destination[k] = v
        return destination


class BatchedFusedEmbeddingBag(BaseEmbedding, FusedOptimizerModule):
    """Pooled lookup; backward applies the optimizer in place (no weight gradient)."""

    def __init__(self, config: GroupedEmbeddingConfig, pg: Optional[dist.ProcessGroup] = None, device: Optional[torch.device] = None,
                 sharding_type: Optional[ShardingType] = None) -> None:
        super().__init__(config, pg, device, pooling_type_to_pooling_mode(config.pooling, sharding_type), fused=True, sharding_type=sharding_type)
        self._optim = EmbeddingFusedOptimizer(config, self._emb_module, pg)

    @property
    def fused_optimizer(self) -> FusedOptimizer:
        return self._optim


class BatchedFusedEmbedding(BaseEmbedding, FusedOptimizerModule):
    """Unpooled (sequence) lookup with the fused optimizer."""

    def __init__(self, config: GroupedEmbeddingConfig, pg: Optional[dist.ProcessGroup] = None, device: Optional[torch.device] = None) -> None:
        super().__init__(config, pg, device, PoolingMode.NONE, fused=True)
        self._optim = EmbeddingFusedOptimizer(config, self._emb_module, pg)

    @property
    def fused_optimizer(self) -> FusedOptimizer:
        return self._optim


class BatchedDenseEmbeddingBag(BaseEmbedding):
    """Pooled lookup that returns a dense weight gradient (data-parallel tables, external optimizers)."""

    def __init__(self, config: GroupedEmbeddingConfig, pg: Optional[dist.ProcessGroup] = None, device: Optional[torch.device] = None,
                 sharding_type: Optional[ShardingType] = None) -> None:
        super().__init__(config, pg, device, pooling_type_to_pooling_mode(config.pooling, sharding_type), fused=False, sharding_type=sharding_type)


class BatchedDenseEmbedding(BaseEmbedding):
    """Unpooled lookup with a dense weight gradient."""

    def __init__(self, config: GroupedEmbeddingConfig, pg: Optional[dist.ProcessGroup] = None, device: Optional[torch.device] = None) -> None:
        super().__init__(config, pg, device, PoolingMode.NONE, fused=False)


def get_state_dict(
    embedding_tables: List[ShardedEmbeddingTable],
    params: List[torch.Tensor],
    pg: Optional[dist.ProcessGroup] = None,
    destination: Optional[Dict[str, Any]] = None,
    prefix: str = "",
) -> Dict[str, Any]:
    """``{prefix}{table}.weight -> ShardedTensor`` (or the plain tensor for unsharded tables)."""
    if destination is None:
        destination = {}
    key_to_local: Dict[str, List[Shard]] = {}
    key_to_global: Dict[str, ShardedTensorMetadata] = {}
    for t, param in zip(embedding_tables, params):
        key = f"{prefix}{t.name}.weight"
        if t.global_metadata is not None and pg is not None:
            gm = copy.deepcopy(t.global_metadata)
            gm.tensor_properties.dtype = param.dtype
            gm.tensor_properties.requires_grad = param.requires_grad
            key_to_global[key] = gm
            key_to_local.setdefault(key, []).append(Shard(param, t.local_metadata))
        else:
            destination[key] = param
    for key, gm in key_to_global.items():
        destination[key] = ShardedTensor._init_from_local_shards_and_global_metadata(
            local_shards=key_to_local[key], sharded_tensor_metadata=gm, process_group=pg,
        )
    return destination
