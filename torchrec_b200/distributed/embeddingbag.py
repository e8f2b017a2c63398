"""Sharded ``EmbeddingBagCollection``.

Tables are grouped by sharding type; each group gets an ``EmbeddingSharding`` that provides its
input dist (KJT redistribution), lookup (TBE kernels) and output dist (pooled all-to-all or
reduce-scatter).  The outputs of all groups are concatenated and permuted back to the table order
of the unsharded module, so ``forward`` returns the same ``KeyedTensor`` an unsharded
``EmbeddingBagCollection`` would.  ``state_dict`` exposes ``embedding_bags.<table>.weight`` as
``ShardedTensor`` whose local shards are views into the kernels' memory.

Counterpart of ``torchrec/distributed/embeddingbag.py`` (``ShardedEmbeddingBagCollection`` ``:454``,
sharder ``:1933``, mean-pooling divisor ``:2253-2340``).
"""
from __future__ import annotations

import copy
from collections import OrderedDict, defaultdict
from typing import Any, Dict, Iterator, List, Optional, Tuple, Type, Union

import torch
import torch.distributed as dist
from torch import nn
from torch.autograd.profiler import record_function
from torch.nn.parallel import DistributedDataParallel

from torchrec_b200.distributed.batched_embedding_kernel import get_state_dict
from torchrec_b200.distributed.embedding_lookup import fused_optimizer_of_lookups
from torchrec_b200.distributed.embedding_sharding import (
    EmbeddingSharding,
    EmbeddingShardingContext,
    EmbeddingShardingInfo,
    KJTListSplitsAwaitable,
)
from torchrec_b200.distributed.embedding_types import (
    BaseEmbeddingSharder,
    EmbeddingComputeKernel,
    KJTList,
    ShardedEmbeddingModule,
)
from torchrec_b200.distributed.sharding.cw_sharding import CwPooledEmbeddingSharding
from torchrec_b200.distributed.sharding.dp_sharding import DpPooledEmbeddingSharding
from torchrec_b200.distributed.sharding.grid_sharding import GridPooledEmbeddingSharding
from torchrec_b200.distributed.sharding.rw_sharding import RwPooledEmbeddingSharding
from torchrec_b200.distributed.sharding.tw_sharding import TwPooledEmbeddingSharding
from torchrec_b200.distributed.sharding.twcw_sharding import TwCwPooledEmbeddingSharding
from torchrec_b200.distributed.sharding.twrw_sharding import TwRwPooledEmbeddingSharding
from torchrec_b200.distributed.types import (
    Awaitable,
    NoWait,
    EmbeddingEvent,
    EmbeddingModuleShardingPlan,
    LazyAwaitable,
    LazyGetItemMixin,
    NullShardedModuleContext,
    ParameterSharding,
    QuantizedCommCodecs,
    ShardedTensor,
    ShardingEnv,
    ShardingEnv2D,
    ShardingType,
)
from torchrec_b200.distributed.utils import (
    add_params_from_parameter_sharding,
    append_prefix,
    convert_to_fbgemm_types,
    maybe_annotate_embedding_event,
    merge_fused_params,
    optimizer_type_to_emb_opt_type,
)
from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig, EmbeddingTableConfig, PoolingType
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection, EmbeddingBagCollectionInterface
from torchrec_b200.ops import sparse_ops as sops
from torchrec_b200.optim.fused import EmptyFusedOptimizer, FusedOptimizerModule
from torchrec_b200.optim.keyed import CombinedOptimizer, KeyedOptimizer
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor, KeyedTensor
from torchrec_b200.streamable import Multistreamable


def _pin_and_move(tensor: torch.Tensor, device: torch.device) -> torch.Tensor:
    if tensor.device == device:
        return tensor
    if device.type == "cuda" and tensor.device.type == "cpu":
        return tensor.pin_memory().to(device=device, non_blocking=True)
    return tensor.to(device=device, non_blocking=True)


def get_device_from_parameter_sharding(ps: ParameterSharding) -> str:
    if ps.sharding_spec is None or not hasattr(ps.sharding_spec, "shards") or not ps.sharding_spec.shards:
        return "cuda" if torch.cuda.is_available() else "cpu"
    return ps.sharding_spec.shards[0].placement.device().type


def replace_placement_with_meta_device(sharding_infos: List[EmbeddingShardingInfo]) -> None:
    """Placements become ``meta`` when a module is sharded on the meta device (plan inspection without memory)."""
    for info in sharding_infos:
        spec = info.param_sharding.sharding_spec
        if spec is None:
            continue
        for shard in spec.shards:
            placement = shard.placement
            if isinstance(placement, str):
                placement = torch.distributed._remote_device(placement)
            shard.placement = torch.distributed._remote_device(f"rank:{placement.rank()}/meta") if placement.rank() is not None else torch.distributed._remote_device("meta")


def create_embedding_bag_sharding(
    sharding_infos: List[EmbeddingShardingInfo], env: ShardingEnv, device: Optional[torch.device] = None,
    permute_embeddings: bool = False, qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None,
) -> EmbeddingSharding[EmbeddingShardingContext, KeyedJaggedTensor, torch.Tensor, torch.Tensor]:
    kind = sharding_infos[0].param_sharding.sharding_type
    if device is not None and device.type == "meta":
        replace_placement_with_meta_device(sharding_infos)
    # sharding type -> (class, takes a codec registry, takes permute_embeddings)
    table = {
        ShardingType.TABLE_WISE.value: (TwPooledEmbeddingSharding, True, False),
        ShardingType.ROW_WISE.value: (RwPooledEmbeddingSharding, True, False),
        ShardingType.DATA_PARALLEL.value: (DpPooledEmbeddingSharding, False, False),
        ShardingType.TABLE_ROW_WISE.value: (TwRwPooledEmbeddingSharding, True, False),
        ShardingType.COLUMN_WISE.value: (CwPooledEmbeddingSharding, True, True),
        ShardingType.TABLE_COLUMN_WISE.value: (TwCwPooledEmbeddingSharding, True, True),
        ShardingType.GRID_SHARD.value: (GridPooledEmbeddingSharding, True, False),
    }
    if kind not in table:
        raise ValueError(f"Sharding type not supported {kind}")
    cls, with_codecs, with_permute = table[kind]
    extra: Dict[str, Any] = {}
    if with_codecs:
        extra["qcomm_codecs_registry"] = qcomm_codecs_registry
    if with_permute:
        extra["permute_embeddings"] = permute_embeddings
    return cls(sharding_infos, env, device, **extra)


def construct_output_kt(embeddings: List[torch.Tensor], embedding_names: List[str], embedding_dims: List[int]) -> KeyedTensor:
    cat_embeddings = embeddings[0] if len(embeddings) == 1 else torch.cat(embeddings, dim=1)
    return KeyedTensor(keys=embedding_names, length_per_key=embedding_dims, values=cat_embeddings, key_dim=1)


class VariableBatchEmbeddingBagCollectionAwaitable(LazyGetItemMixin[str, torch.Tensor], LazyAwaitable[KeyedTensor]):
    """Output awaitable for variable batch per feature: flat per-feature outputs are expanded to the
    full batch through the inverse indices."""

    def __init__(self, awaitables: List[Awaitable[torch.Tensor]], inverse_indices: Tuple[List[str], torch.Tensor],
                 inverse_indices_permute_indices: Optional[torch.Tensor], batch_size_per_feature_pre_a2a: List[int],
                 uncombined_embedding_dims: List[int], embedding_names: List[str], embedding_dims: List[int],
                 permute_op: Optional[nn.Module], module_fqn: Optional[str] = None, sharding_types: Optional[List[str]] = None) -> None:
        super().__init__()
        self._awaitables = awaitables
        self._inverse_indices = inverse_indices
        self._inverse_indices_permute_indices = inverse_indices_permute_indices
        self._batch_size_per_feature_pre_a2a = batch_size_per_feature_pre_a2a
        self._uncombined_embedding_dims = uncombined_embedding_dims
        self._embedding_names = embedding_names
        self._embedding_dims = embedding_dims
        self._permute_op = permute_op

    def _wait_impl(self) -> KeyedTensor:
        embeddings = [w.wait() for w in self._awaitables]
        flat = torch.cat([e.view(-1) for e in embeddings])
        inv = self._inverse_indices[1]
        if self._inverse_indices_permute_indices is not None:
            inv = torch.index_select(inv, 0, self._inverse_indices_permute_indices)
        values = sops.vbe_expand(flat, inv, self._batch_size_per_feature_pre_a2a, self._uncombined_embedding_dims)
        if self._permute_op is not None:
            values = self._permute_op(values)
        return KeyedTensor(keys=self._embedding_names, length_per_key=self._embedding_dims, values=values, key_dim=1)


class EmbeddingBagCollectionAwaitable(LazyGetItemMixin[str, torch.Tensor], LazyAwaitable[KeyedTensor]):
    def __init__(self, awaitables: List[Awaitable[torch.Tensor]], embedding_dims: List[int], embedding_names: List[str],
                 module_fqn: Optional[str] = None, sharding_types: Optional[List[str]] = None) -> None:
        super().__init__()
        self._awaitables = awaitables
        self._embedding_dims = embedding_dims
        self._embedding_names = embedding_names
        self._module_fqn = module_fqn
        self._sharding_types = sharding_types

    def _wait_impl(self) -> KeyedTensor:
        embeddings = []
        for i, w in enumerate(self._awaitables):
            with maybe_annotate_embedding_event(EmbeddingEvent.OUTPUT_DIST_WAIT, self._module_fqn, self._sharding_types[i] if self._sharding_types else None):
                embeddings.append(w.wait())
        return construct_output_kt(embeddings, self._embedding_names, self._embedding_dims)


class EmbeddingBagCollectionContext(Multistreamable):
    def __init__(self, sharding_contexts: Optional[List[Optional[EmbeddingShardingContext]]] = None,
                 inverse_indices: Optional[Tuple[List[str], torch.Tensor]] = None, variable_batch_per_feature: bool = False,
                 divisor: Optional[torch.Tensor] = None) -> None:
        super().__init__()
        self.sharding_contexts: List[Optional[EmbeddingShardingContext]] = sharding_contexts if sharding_contexts else []
        self.inverse_indices = inverse_indices
        self.variable_batch_per_feature = variable_batch_per_feature
        self.divisor = divisor
        self.engine_handle = None  # set when the fused sparse engine distributed this batch

    def record_stream(self, stream: torch.Stream) -> None:
        if self.engine_handle is not None:
            self.engine_handle.record_stream(stream)
        for ctx in self.sharding_contexts:
            if ctx:
                ctx.record_stream(stream)
        if self.inverse_indices is not None and self.inverse_indices[1].is_cuda:
            self.inverse_indices[1].record_stream(stream)
        if self.divisor is not None and self.divisor.is_cuda:
            self.divisor.record_stream(stream)


def _create_mean_pooling_divisor(lengths: torch.Tensor, keys: List[str], offsets: torch.Tensor, stride: int,
                                 dim_per_key: torch.Tensor, mean_features: List[str], embedding_names: List[str],
                                 embedding_dims: List[int], kjt_key_indices: Dict[str, int], kt_key_ordering: torch.Tensor,
                                 weights: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``[B, sum(D)]`` divisor: the bag length for MEAN features of row-split tables, 1 elsewhere."""
    with record_function("## ebc create mean pooling callback ##"):
        batch_size = stride
        if weights is not None:
            lengths = sops.segment_sum_csr(1, offsets.to(torch.int64), weights)
        lengths = lengths.clone().to(torch.float32)
        mean_set = set(mean_features)
        for feature in keys:
            if feature not in mean_set:
                i = kjt_key_indices[feature] * batch_size
                lengths[i: i + batch_size] = 1
        # rows of `lengths` follow the (permuted) input keys; the divisor must follow the output embedding order
        if len(embedding_names) != len(keys) or [n.split("@")[0] for n in embedding_names] != list(keys):
            lengths = torch.index_select(lengths.reshape(-1, batch_size), 0, kt_key_ordering).reshape(-1)
        lengths = lengths.reshape(-1, batch_size).T
        divisor = torch.repeat_interleave(lengths, dim_per_key, dim=1, output_size=sum(embedding_dims))
        return (divisor + 1e-6).detach()


def _apply_mean_pooling(keyed_tensor: KeyedTensor, divisor: torch.Tensor) -> KeyedTensor:
    with record_function("## ebc apply mean pooling ##"):
        return KeyedTensor(keys=keyed_tensor.keys(), values=keyed_tensor.values() / divisor.to(keyed_tensor.values().dtype),
                           length_per_key=keyed_tensor.length_per_key(), key_dim=1)


class ShardedTableStateMixin:
    """Parameters and checkpoint views of the tables of a sharded embedding module (pooled or unpooled): what
    ``named_parameters`` / ``state_dict`` / ``load_state_dict`` see.  The module provides ``_TABLE_ATTR``, ``_table_configs()``,
    ``_sharding_types``, ``_lookups``, ``module_sharding_plan``, ``_env``, ``_device`` and ``_output_dtensor``."""

    # ---- construction steps shared by the pooled and the unpooled module ---------------------------------
    def _replicate_data_parallel_lookups(self, dp_sharding_cls: type) -> None:
        """Lookups of replicated (data-parallel) tables get their dense gradient all-reduced by DDP."""
        pg = self._env.process_group
        if pg is None or dist.get_backend(pg) == "fake":
            return
        on_cuda = self._device is not None and self._device.type == "cuda"
        for i, sharding in enumerate(self._embedding_shardings):
            if isinstance(sharding, dp_sharding_cls):
                self._lookups[i] = DistributedDataParallel(
                    module=self._lookups[i], device_ids=[self._device] if on_cuda else None, process_group=pg,
                    gradient_as_bucket_view=True, broadcast_buffers=True, static_graph=True,
                )

    def _gather_fused_optimizers(self) -> CombinedOptimizer:
        """One optimizer over the in-backward optimizers of all kernels, with keys ``<tables attr>.<table>.weight``."""
        prefix = self._TABLE_ATTR + "."
        found = []
        for _, lookup in self._unwrapped_lookups():
            for kernel in lookup.modules():
                if isinstance(kernel, FusedOptimizerModule):
                    opt = kernel.fused_optimizer
                    opt.params = {prefix + key: weight for key, weight in opt.params.items()}
                    found.append(("", opt))
        if getattr(self, "_output_dtensor", False):
            for _, opt in found:
                self._optimizer_states_as_dtensor(opt)
        return CombinedOptimizer(found)

    def _optimizer_states_as_dtensor(self, opt) -> None:
        """With ``env.output_dtensor`` the in-backward optimizer states leave as ``DTensor`` s like the tables do: every sharded state
        is re-wrapped around the SAME local shard tensors (views of the kernel's state memory), with their offsets, over the
        sharding group's mesh; row-wise states (one value per row) and row-split tables shard dim 0, column-split 2-D states dim 1."""
        try:
            from torch.distributed.device_mesh import DeviceMesh
            from torch.distributed.tensor import DTensor, Replicate, Shard

            from torchrec_b200.distributed.shards_wrapper import LocalShardsWrapper
        except Exception:
            return
        pg = self._env.sharding_pg if isinstance(self._env, ShardingEnv2D) else self._env.process_group
        if pg is None:
            return
        mesh = getattr(self._env, "device_mesh", None)
        if mesh is None or mesh.ndim != 1:
            mesh = DeviceMesh.from_group(pg, self._device.type if self._device is not None else "cpu")
        row_kinds = (ShardingType.ROW_WISE.value, ShardingType.TABLE_ROW_WISE.value, ShardingType.GRID_SHARD.value)
        col_kinds = (ShardingType.COLUMN_WISE.value, ShardingType.TABLE_COLUMN_WISE.value)
        for per_param in opt.state.values():
            for key, value in list(per_param.items()):
                if not isinstance(value, ShardedTensor):
                    continue
                table = key.rsplit(".", 1)[0].split(".")[-1]
                kind = self.module_sharding_plan[table].sharding_type if table in self.module_sharding_plan else None
                shards = value.local_shards()
                size = value.size()
                if len(size) == 1 or kind in row_kinds:
                    placements = (Shard(0),)
                elif kind in col_kinds:
                    placements = (Shard(1),)
                else:
                    placements = (Replicate(),)
                wrapper = LocalShardsWrapper([s.tensor for s in shards], [tuple(int(x) for x in s.metadata.shard_offsets) for s in shards])
                stride = (int(size[1]), 1) if len(size) == 2 else (1,)
                per_param[key] = DTensor.from_local(wrapper, mesh, placements, run_check=False, shape=torch.Size(size), stride=stride)

    # ---- torch state: parameters and state dict -----------------------------------------------------
    def _unwrapped_lookups(self):
        for sharding_type, lookup in zip(self._sharding_types, self._lookups):
            yield sharding_type, (lookup.module if isinstance(lookup, DistributedDataParallel) else lookup)

    def _initialize_torch_state(self) -> None:
        """Register ``embedding_bags.<table>.weight`` and build the checkpoint view of every model-parallel table: a
        ``ShardedTensor``, or (``env.output_dtensor``) a ``DTensor`` whose local tensor wraps this rank's shards."""
        holder = nn.ModuleDict()
        setattr(self, self._TABLE_ATTR, holder)
        self._name_to_table_size: Dict[str, Tuple[int, int]] = {c.name: (c.num_embeddings, c.embedding_dim) for c in self._table_configs()}
        plan = self.module_sharding_plan
        model_parallel = [t for t, ps in plan.items() if ps.sharding_type != ShardingType.DATA_PARALLEL.value]
        self._model_parallel_name_to_local_shards: Dict[str, List[Any]] = OrderedDict((t, []) for t in model_parallel)
        self._model_parallel_name_to_sharded_tensor: Dict[str, Any] = OrderedDict()
        # local shards of every table, straight views into the kernels' memory
        for sharding_type, lookup in self._unwrapped_lookups():
            for emb in lookup.emb_modules:
                if sharding_type == ShardingType.DATA_PARALLEL.value:
                    self._register_data_parallel_tables(holder, emb)
                    continue
                for table, weight in zip(emb.config.embedding_tables, emb.split_embedding_weights()):
                    self._model_parallel_name_to_local_shards[table.name].append((table, weight))
        pg = self._env.sharding_pg if isinstance(self._env, ShardingEnv2D) else self._env.process_group
        for name in model_parallel:
            local = self._model_parallel_name_to_local_shards[name]
            slot = nn.Module()
            holder[name] = slot
            slot.register_parameter("weight", self._local_parameter(local))
            if plan[name].compute_kernel != EmbeddingComputeKernel.DENSE.value:
                slot.weight._in_backward_optimizers = [EmptyFusedOptimizer()]  # updated inside the kernel's backward: dense optimizers skip it
            if pg is not None:
                self._model_parallel_name_to_sharded_tensor[name] = self._checkpoint_view(name, local, pg)

        def post_state_dict_hook(module, destination, prefix, _local_metadata) -> None:
            for name, view in module._model_parallel_name_to_sharded_tensor.items():
                key = f"{prefix}{module._TABLE_ATTR}.{name}.weight"
                if view is not None:
                    destination[key] = view
                elif not module._model_parallel_name_to_local_shards.get(name):
                    destination.pop(key, None)

        self._register_state_dict_hook(post_state_dict_hook)
        self._register_load_state_dict_pre_hook(self._pre_load_state_dict_hook, with_module=True)
        self.reset_parameters()

    @staticmethod
    def _register_data_parallel_tables(holder: nn.ModuleDict, emb) -> None:
        """Data-parallel tables are ordinary parameters: ``[rows, cols]`` views into the dense kernel's flat buffer."""
        from torchrec_b200.distributed.batched_embedding_kernel import TableBatchedEmbeddingSlice

        flat, bounds = emb.emb_module.weights, emb.emb_module.weights_offsets
        for i, table in enumerate(emb.config.embedding_tables):
            slot = nn.Module()
            slot.register_parameter("weight", TableBatchedEmbeddingSlice(flat, bounds[i], bounds[i + 1], table.local_rows, table.local_cols))
            holder[table.name] = slot

    def _local_parameter(self, local: List[Tuple[Any, torch.Tensor]]) -> nn.Parameter:
        """What ``named_parameters`` shows for a table: the shard itself when the rank holds one, the column shards side by
        side when it holds several of equal height, an empty parameter when it holds none."""
        if not local:
            dev = self._device if self._device is not None else torch.device("cpu")
            return nn.Parameter(torch.empty(0, device=dev), requires_grad=False)
        if len(local) == 1:
            return _ViewParameter(local[0][1])
        heights = {w.shape[0] for _, w in local}
        joined = torch.cat([w for _, w in local], dim=1) if len(heights) == 1 else local[0][1]
        return nn.Parameter(joined, requires_grad=False)

    def _checkpoint_view(self, name: str, local: List[Tuple[Any, torch.Tensor]], pg):
        rows, cols = self._name_to_table_size[name]
        if self._output_dtensor:
            view = self._dtensor_view(name, local, pg, rows, cols)
            if view is not None:
                return view
        if local:
            return get_state_dict([t for t, _ in local], [w for _, w in local], pg=pg)[f"{name}.weight"]
        # a rank without a shard of the table still takes part in the ShardedTensor
        from torchrec_b200.distributed.types import ShardedTensorMetadata, TensorProperties

        meta = ShardedTensorMetadata(shards_metadata=copy.deepcopy(self.module_sharding_plan[name].sharding_spec.shards), size=torch.Size([rows, cols]),
                                     tensor_properties=TensorProperties(dtype=torch.float32))
        try:
            return ShardedTensor._init_from_local_shards_and_global_metadata(local_shards=[], sharded_tensor_metadata=meta, process_group=pg)
        except Exception:
            return None

    def _dtensor_view(self, name: str, local: List[Tuple[Any, torch.Tensor]], pg, rows: int, cols: int):
        """``DTensor`` over a 1-D mesh of the sharding group.  Its local tensor is a ``LocalShardsWrapper`` holding this rank's
        shards with their (row, column) offsets, which is what distributed checkpointing reads; the placement names the split
        dimension (rows for row-wise kinds, columns for column-wise kinds, replicate for table-wise)."""
        try:
            from torch.distributed.device_mesh import DeviceMesh
            from torch.distributed.tensor import DTensor, Replicate, Shard

            from torchrec_b200.distributed.shards_wrapper import LocalShardsWrapper
        except Exception:
            return None
        mesh = getattr(self._env, "device_mesh", None)
        if mesh is None or mesh.ndim != 1:
            dev_type = self._device.type if self._device is not None else "cpu"
            mesh = DeviceMesh.from_group(pg, dev_type)
        kind = self.module_sharding_plan[name].sharding_type
        if kind in (ShardingType.ROW_WISE.value, ShardingType.TABLE_ROW_WISE.value, ShardingType.GRID_SHARD.value):
            placements = (Shard(0),)
        elif kind in (ShardingType.COLUMN_WISE.value, ShardingType.TABLE_COLUMN_WISE.value):
            placements = (Shard(1),)
        else:
            placements = (Replicate(),)
        shards = [w for _, w in local]
        offsets = [tuple(int(x) for x in t.local_metadata.shard_offsets) for t, _ in local]
        wrapper = LocalShardsWrapper(shards, offsets)
        return DTensor.from_local(wrapper, mesh, placements, run_check=False, shape=torch.Size([rows, cols]), stride=(cols, 1))

    @staticmethod
    def _pre_load_state_dict_hook(self, state_dict, prefix, *args) -> None:
        """Copy incoming (sharded or full) tensors into the local shard views, then hand nn.Module the
        local parameter itself so that its own copy is a no-op."""
        for name in list(self._model_parallel_name_to_local_shards.keys()):
            key = f"{prefix}{self._TABLE_ATTR}.{name}.weight"
            if key not in state_dict:
                continue
            src = state_dict[key]
            local = self._model_parallel_name_to_local_shards[name]
            if isinstance(src, ShardedTensor):
                src_shards = src.local_shards()
                for t, w in local:
                    for s in src_shards:
                        if list(s.metadata.shard_offsets) == list(t.local_metadata.shard_offsets) and list(s.metadata.shard_sizes) == list(t.local_metadata.shard_sizes):
                            w.detach().copy_(s.tensor)
                            break
                    else:
                        raise RuntimeError(f"no matching shard for {name} at offsets {t.local_metadata.shard_offsets}")
            elif type(src).__name__ == "DTensor":
                inner = src.to_local()
                pieces = list(zip(inner.local_shards(), inner.local_offsets())) if hasattr(inner, "local_shards") else []
                for t, w in local:
                    want = tuple(int(x) for x in t.local_metadata.shard_offsets)
                    match = [piece for piece, at in pieces if tuple(int(x) for x in at) == want and tuple(piece.shape) == tuple(w.shape)]
                    if not match:
                        raise RuntimeError(f"no matching shard for {name} at offsets {want}")
                    if match[0].data_ptr() != w.data_ptr():
                        w.detach().copy_(match[0])
            elif isinstance(src, torch.Tensor):
                rows, cols = self._name_to_table_size[name]
                if tuple(src.shape) == (rows, cols):
                    for t, w in local:
                        ro, co = t.local_metadata.shard_offsets
                        rs, cs = t.local_metadata.shard_sizes
                        w.detach().copy_(src[ro: ro + rs, co: co + cs])
                elif local and tuple(src.shape) == tuple(local[0][1].shape):
                    local[0][1].detach().copy_(src)
            state_dict[key] = getattr(self, self._TABLE_ATTR)[name].weight.detach()



class ShardedEmbeddingBagCollection(
    ShardedTableStateMixin,
    ShardedEmbeddingModule[KJTList, List[torch.Tensor], KeyedTensor, EmbeddingBagCollectionContext],
    FusedOptimizerModule,
):
    """Sharded counterpart of ``EmbeddingBagCollection``; built by ``EmbeddingBagCollectionSharder``."""

    _TABLE_ATTR: str = "embedding_bags"  # name of the ModuleDict that holds ``<table>.weight``

    def _table_configs(self):
        return self._embedding_bag_configs

    def __init__(
        self,
        module: EmbeddingBagCollectionInterface,
        table_name_to_parameter_sharding: Dict[str, ParameterSharding],
        env: ShardingEnv,
        fused_params: Optional[Dict[str, Any]] = None,
        device: Optional[torch.device] = None,
        qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None,
        module_fqn: Optional[str] = None,
    ) -> None:
        super().__init__(qcomm_codecs_registry=qcomm_codecs_registry)
        self._module_fqn = module_fqn
        self._embedding_bag_configs: List[EmbeddingBagConfig] = module.embedding_bag_configs()
        self._table_names: List[str] = [c.name for c in self._embedding_bag_configs]
        self._table_name_to_config: Dict[str, EmbeddingBagConfig] = {c.name: c for c in self._embedding_bag_configs}
        self.module_sharding_plan: EmbeddingModuleShardingPlan = EmbeddingModuleShardingPlan(
            {t: ps for t, ps in table_name_to_parameter_sharding.items() if t in self._table_names}
        )
        self._env = env
        self._output_dtensor: bool = env.output_dtensor
        self.sharding_type_to_sharding_infos = self.create_grouped_sharding_infos(module, table_name_to_parameter_sharding, "embedding_bags.", fused_params)
        self._sharding_types: List[str] = list(self.sharding_type_to_sharding_infos.keys())
        self._embedding_shardings: List[EmbeddingSharding] = [
            create_embedding_bag_sharding(infos, env, device, permute_embeddings=True, qcomm_codecs_registry=self.qcomm_codecs_registry)
            for infos in self.sharding_type_to_sharding_infos.values()
        ]
        self._is_weighted: bool = module.is_weighted()
        self._device = device
        self._lookups: List[nn.Module] = []
        self._create_lookups()
        self._reset_dist_layout()
        self._replicate_data_parallel_lookups(DpPooledEmbeddingSharding)
        self._initialize_torch_state()
        self._optim: CombinedOptimizer = self._gather_fused_optimizers()
        # mean pooling for row-split tables is applied after the reduction
        self._has_mean_pooling_callback: bool = PoolingType.MEAN.value in self._pooling_type_to_rs_features()
        # fused sparse engine (peer-memory input dist + lookup + output hand-over): built on the first batch, collectively
        self._engine_state: str = "auto"  # "auto" -> "on" | "off"
        self._engine = None
        self._dim_per_key: Optional[torch.Tensor] = None
        self._kjt_key_indices: Dict[str, int] = {}
        self._kt_key_ordering: Optional[torch.Tensor] = None

    def _reset_dist_layout(self) -> None:
        """Everything the first batch fills in (the key order of the incoming KJT decides it): dist modules, output names and
        dims, feature order, the column permutation back to table order."""
        for name in ("_input_dists", "_output_dists", "_embedding_names", "_embedding_dims", "_feature_splits", "_features_order",
                     "_uncombined_embedding_names", "_uncombined_embedding_dims"):
            setattr(self, name, [])
        self._inverse_indices_permute_indices: Optional[torch.Tensor] = None
        self._permute_op: Optional[nn.Module] = None
        self._has_uninitialized_input_dist, self._has_features_permute = True, True

    # ---- plan -> sharding infos ------------------------------------------------------------------
    @classmethod
    def create_grouped_sharding_infos(cls, module, table_name_to_parameter_sharding: Dict[str, ParameterSharding], prefix: str,
                                      fused_params: Optional[Dict[str, Any]], suffix: Optional[str] = "weight") -> Dict[str, List[EmbeddingShardingInfo]]:
        """``{sharding type: [one EmbeddingShardingInfo per table]}`` in the order the tables appear in the module.  A feature
        that feeds two tables gets the embedding name ``feature@table`` so that output columns stay distinguishable."""
        configs = list(module.embedding_bag_configs())
        for cfg in configs:
            cfg.feature_names = cfg.feature_names or [cfg.name]
        uses: Dict[str, int] = defaultdict(int)
        for cfg in configs:
            for f in cfg.feature_names:
                uses[f] += 1
        tensors: Dict[str, Any] = dict(module.state_dict())
        tensors.update(dict(module.named_parameters()))  # parameters win: they carry the optimizer annotations
        valid_kernels = {k.value for k in EmbeddingComputeKernel}
        grouped: Dict[str, List[EmbeddingShardingInfo]] = defaultdict(list)
        for cfg in configs:
            assert cfg.name in table_name_to_parameter_sharding, f"{cfg.name} not in table_name_to_parameter_sharding"
            ps = table_name_to_parameter_sharding[cfg.name]
            if ps.compute_kernel not in valid_kernels:
                raise ValueError(f"Compute kernel not supported {ps.compute_kernel}")
            key = prefix + cfg.name + ("" if suffix is None else f".{suffix}")
            assert key in tensors, f"{key} is neither a parameter nor a state-dict entry of the module"
            param = tensors[key]
            table = EmbeddingTableConfig(
                num_embeddings=cfg.num_embeddings, embedding_dim=cfg.embedding_dim, name=cfg.name, data_type=cfg.data_type,
                feature_names=list(cfg.feature_names), pooling=cfg.pooling, is_weighted=module.is_weighted(), has_feature_processor=False,
                embedding_names=[f"{f}@{cfg.name}" if uses[f] > 1 else f for f in cfg.feature_names],
                weight_init_max=cfg.weight_init_max, weight_init_min=cfg.weight_init_min, init_fn=cfg.init_fn,
                num_embeddings_post_pruning=getattr(cfg, "num_embeddings_post_pruning", None),
                total_num_buckets=getattr(cfg, "total_num_buckets", None), use_virtual_table=getattr(cfg, "use_virtual_table", False),
            )
            grouped[ps.sharding_type].append(
                EmbeddingShardingInfo(embedding_config=table, param_sharding=ps, param=param, fused_params=cls._table_fused_params(param, ps, fused_params or {}))
            )
        return grouped

    @staticmethod
    def _table_fused_params(param, ps: ParameterSharding, module_fused_params: Dict[str, Any]) -> Dict[str, Any]:
        """Kernel options of one table: module-level options, overridden by the optimizer attached to the parameter
        (``apply_optimizer_in_backward``), then by what the plan fixed for this table."""
        classes = getattr(param, "_optimizer_classes", [None])
        kwargs = getattr(param, "_optimizer_kwargs", [{}])
        assert len(classes) == 1 and len(kwargs) == 1, "Only support 1 optimizer per table"
        from_optimizer = copy.deepcopy(kwargs[0])
        if classes[0]:
            from_optimizer["optimizer"] = optimizer_type_to_emb_opt_type(classes[0])
        merged = merge_fused_params(module_fused_params, from_optimizer)
        return convert_to_fbgemm_types(add_params_from_parameter_sharding(merged, ps))

    def _pooling_type_to_rs_features(self) -> Dict[str, List[str]]:
        out: Dict[str, List[str]] = defaultdict(list)
        for sharding_type, infos in self.sharding_type_to_sharding_infos.items():
            if sharding_type in (ShardingType.ROW_WISE.value, ShardingType.TABLE_ROW_WISE.value, ShardingType.GRID_SHARD.value):
                for info in infos:
                    out[info.embedding_config.pooling.value].extend(info.embedding_config.feature_names)
        return out

    def reset_parameters(self) -> None:
        if self._device is not None and self._device.type == "meta":
            return
        # data-parallel tables start identical on every rank: DDP broadcasts rank 0's parameters at construction
        return

    # ---- parameters / optimizer ---------------------------------------------------------------------
    def named_parameters(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True) -> Iterator[Tuple[str, nn.Parameter]]:
        for name, m in getattr(self, self._TABLE_ATTR).items():
            yield append_prefix(prefix, f"{self._TABLE_ATTR}.{name}.weight"), m.weight

    def sharded_parameter_names(self, prefix: str = "") -> Iterator[str]:
        for name in self._model_parallel_name_to_local_shards.keys():
            yield append_prefix(prefix, f"{self._TABLE_ATTR}.{name}.weight")

    @property
    def fused_optimizer(self) -> KeyedOptimizer:
        return self._optim

    @property
    def shardings(self) -> Dict[str, EmbeddingSharding]:
        return dict(zip(self._sharding_types, self._embedding_shardings))

    @property
    def unsharded_module_type(self) -> Type[EmbeddingBagCollection]:
        return EmbeddingBagCollection

    def create_context(self) -> EmbeddingBagCollectionContext:
        return EmbeddingBagCollectionContext()

    # ---- building the three stages --------------------------------------------------------------------
    def _create_lookups(self) -> None:
        for sharding in self._embedding_shardings:
            self._lookups.append(sharding.create_lookup())

    def _create_input_dist(self, input_feature_names: List[str]) -> None:
        """One input dist per sharding; the incoming KJT is permuted only if its key order differs from the shardings'."""
        per_sharding = [sh.feature_names() for sh in self._embedding_shardings]
        self._input_dists.extend(sh.create_input_dist() for sh in self._embedding_shardings)
        self._feature_splits.extend(len(names) for names in per_sharding)
        wanted = [f for names in per_sharding for f in names]
        self._has_features_permute = wanted != list(input_feature_names)
        if self._has_features_permute:
            position = {f: i for i, f in reversed(list(enumerate(input_feature_names)))}  # first occurrence wins
            self._features_order.extend(position[f] for f in wanted)
            dev = torch.device("cpu") if self._device is None or self._device.type == "meta" else self._device
            self.register_buffer("_features_order_tensor", torch.tensor(self._features_order, device=dev, dtype=torch.int32), persistent=False)

    def _create_output_dist(self) -> None:
        """One output dist per sharding, plus the column permutation that restores the unsharded module's embedding order."""
        for sh in self._embedding_shardings:
            self._output_dists.append(sh.create_output_dist(device=self._device))
            for attr, values in (("_embedding_names", sh.embedding_names()), ("_embedding_dims", sh.embedding_dims()),
                                 ("_uncombined_embedding_names", sh.uncombined_embedding_names()),
                                 ("_uncombined_embedding_dims", sh.uncombined_embedding_dims())):
                getattr(self, attr).extend(values)
        module_order = [n for names in _embedding_names_by_table(self._embedding_bag_configs) for n in names]
        if module_order == self._embedding_names:
            return
        from torchrec_b200.distributed.sharding.cw_sharding import PermutePooledEmbeddingsSplit

        order = [self._embedding_names.index(n) for n in module_order]
        self._pre_names, self._pre_dims = list(self._embedding_names), list(self._embedding_dims)
        self._permute_op = PermutePooledEmbeddingsSplit(self._pre_dims, order, device=self._device)
        self._embedding_names, self._embedding_dims = module_order, [self._pre_dims[i] for i in order]

    def _init_mean_pooling_callback(self, input_feature_names: List[str]) -> None:
        keys = [input_feature_names[i] for i in self._features_order] if self._features_order else list(input_feature_names)
        self._kjt_key_indices = {k: i for i, k in enumerate(keys)}
        dev = self._device if self._device is not None else torch.device("cpu")
        self._dim_per_key = torch.tensor(self._embedding_dims, device=dev)
        # embedding name -> feature name ("f@table" -> "f")
        feat_of = [n.split("@")[0] for n in self._embedding_names]
        self._kt_key_ordering = torch.tensor([self._kjt_key_indices[f] for f in feat_of], device=dev)

    # ---- the three stages -------------------------------------------------------------------------------
    # ---- fused sparse engine ---------------------------------------------------------------------------
    def disable_fused_engine(self) -> None:
        """Wrappers that transform the distributed KJT between input dist and lookup (feature processors, managed
        collision, pruning) need the classic three-stage path."""
        self._engine_state, self._engine = "off", None

    def _fused_engine(self):
        if self._engine_state == "auto":
            self._engine = self._build_fused_engine()
            self._engine_state = "on" if self._engine is not None else "off"
        return self._engine

    def _build_fused_engine(self):
        """All ranks take the same decision: it depends on the plan, the environment and one collective agreement."""
        from torchrec_b200.distributed.fbgemm_qcomm_codec import CastCodec
        from torchrec_b200.distributed.fused_sparse_engine import FusedSparseEngine
        from torchrec_b200.distributed.peer_memory import PeerGroup
        from torchrec_b200.distributed.types import CommOp

        dev = self._device
        if dev is None or dev.type != "cuda" or isinstance(self._env, ShardingEnv2D):
            return None
        allowed = {ShardingType.TABLE_WISE.value, ShardingType.COLUMN_WISE.value, ShardingType.TABLE_COLUMN_WISE.value,
                   ShardingType.ROW_WISE.value, ShardingType.TABLE_ROW_WISE.value, ShardingType.GRID_SHARD.value}
        if not self._sharding_types or any(t not in allowed for t in self._sharding_types):
            return None
        fused = (EmbeddingComputeKernel.FUSED, EmbeddingComputeKernel.FUSED_UVM, EmbeddingComputeKernel.FUSED_UVM_CACHING)
        out_dtypes = set()
        for sh, lk in zip(self._embedding_shardings, self._lookups):
            if isinstance(lk, DistributedDataParallel) or getattr(lk, "_feature_processor", None) is not None:
                return None
            for groups in sh._grouped_embedding_configs_per_rank:
                for g in groups:
                    if g.compute_kernel not in fused or g.has_feature_processor:
                        return None
                    if g.is_weighted and g.pooling.value == PoolingType.MEAN.value:
                        return None
            for emb in lk.emb_modules:
                out_dtypes.add(emb.emb_module.output_dtype)
        if len(out_dtypes) > 1:
            return None
        out_dtype = out_dtypes.pop() if out_dtypes else torch.float32
        stage_dtype, grad_dtype = out_dtype, torch.float32
        reg = self.qcomm_codecs_registry or {}
        for op in (CommOp.POOLED_EMBEDDINGS_ALL_TO_ALL.name, CommOp.POOLED_EMBEDDINGS_REDUCE_SCATTER.name):
            codecs = reg.get(op)
            if codecs is None:
                continue
            fwd, bwd = codecs.forward, codecs.backward
            stage_dtype = fwd.quantized_dtype if isinstance(fwd, CastCodec) and fwd.quantized_dtype != torch.float32 else (torch.float16 if not isinstance(fwd, CastCodec) else stage_dtype)
            grad_dtype = bwd.quantized_dtype if isinstance(bwd, CastCodec) and bwd.quantized_dtype != torch.float32 else (torch.bfloat16 if not isinstance(bwd, CastCodec) else grad_dtype)
        pg = self._env.process_group
        peer = PeerGroup.get(pg, dev)
        if peer is None:
            return None
        try:
            return FusedSparseEngine(peer, self._embedding_bag_configs, self._embedding_shardings, self._lookups, out_dtype, stage_dtype, grad_dtype)
        except AssertionError as e:
            import warnings

            warnings.warn(f"fused sparse engine not used for this module: {e}")
            return None

    def _engine_names_dims(self) -> Tuple[List[str], List[int]]:
        names = [n for ns in _embedding_names_by_table(self._embedding_bag_configs) for n in ns]
        dims = [cfg.embedding_dim for cfg in self._embedding_bag_configs for _ in cfg.feature_names]
        return names, dims

    def _engine_output(self, ctx: EmbeddingBagCollectionContext) -> LazyAwaitable[KeyedTensor]:
        out = self._engine.lookup(ctx.engine_handle)
        names, dims = self._engine_names_dims()
        return EmbeddingBagCollectionAwaitable(awaitables=[NoWait(out)], embedding_dims=dims, embedding_names=names,
                                               module_fqn=self._module_fqn, sharding_types=None)

    def input_dist(self, ctx: EmbeddingBagCollectionContext, features: KeyedJaggedTensor) -> Awaitable[Awaitable[KJTList]]:
        ctx.variable_batch_per_feature = features.variable_stride_per_key()
        ctx.inverse_indices = features.inverse_indices_or_none()
        engine = self._fused_engine() if self._engine_state != "off" else None
        if engine is not None and engine.accepts(features):
            ctx.engine_handle = engine.input_dist(features)
            return NoWait(NoWait(EngineDistInput(ctx.engine_handle)))
        if self._has_uninitialized_input_dist:
            self._first_batch_setup(features, ctx)
        with torch.no_grad():
            if self._has_features_permute:
                features = features.permute(self._features_order, self._features_order_tensor)
            if self._has_mean_pooling_callback:
                ctx.divisor = self._mean_divisor(features)
            requests = []
            for dist_module, shard_features, sharding_type in zip(self._input_dists, features.split(self._feature_splits), self._sharding_types):
                with maybe_annotate_embedding_event(EmbeddingEvent.KJT_SPLITS_DIST, self._module_fqn, sharding_type):
                    requests.append(dist_module(shard_features))
                ctx.sharding_contexts.append(EmbeddingShardingContext(
                    batch_size_per_feature_pre_a2a=shard_features.stride_per_key(),
                    variable_batch_per_feature=shard_features.variable_stride_per_key()))
            return KJTListSplitsAwaitable(requests, ctx, self._module_fqn, self._sharding_types)

    def _first_batch_setup(self, features: KeyedJaggedTensor, ctx: EmbeddingBagCollectionContext) -> None:
        self._create_input_dist(features.keys())
        self._has_uninitialized_input_dist = False
        if not self._output_dists:
            self._create_output_dist()
        if ctx.variable_batch_per_feature and ctx.inverse_indices is not None:
            self._create_inverse_indices_permute_indices(ctx.inverse_indices)
        if self._has_mean_pooling_callback:
            self._init_mean_pooling_callback(features.keys())

    def _mean_divisor(self, features: KeyedJaggedTensor) -> torch.Tensor:
        return _create_mean_pooling_divisor(
            lengths=features.lengths(), keys=features.keys(), offsets=features.offsets(), stride=features.stride(),
            dim_per_key=self._dim_per_key, mean_features=self._pooling_type_to_rs_features()[PoolingType.MEAN.value],
            embedding_names=self._embedding_names, embedding_dims=self._embedding_dims, kjt_key_indices=self._kjt_key_indices,
            kt_key_ordering=self._kt_key_ordering, weights=features.weights_or_none() if self._is_weighted else None)

    def _create_inverse_indices_permute_indices(self, inverse_indices: Optional[Tuple[List[str], torch.Tensor]]) -> None:
        assert inverse_indices is not None, "inverse indices must be provided from KJT if using variable batch size per feature."
        index_per_name = {name: i for i, name in enumerate(inverse_indices[0])}
        permute_indices = [index_per_name[n.split("@")[0]] for n in self._uncombined_embedding_names]
        if len(permute_indices) != len(index_per_name) or permute_indices != sorted(permute_indices):
            self._inverse_indices_permute_indices = _pin_and_move(torch.tensor(permute_indices), inverse_indices[1].device)

    def compute(self, ctx: EmbeddingBagCollectionContext, dist_input: KJTList) -> List[torch.Tensor]:
        if isinstance(dist_input, EngineDistInput):
            return [self._engine.lookup(ctx.engine_handle)]
        return [lookup(features) for lookup, features in zip(self._lookups, dist_input)]

    def output_dist(self, ctx: EmbeddingBagCollectionContext, output: List[torch.Tensor]) -> LazyAwaitable[KeyedTensor]:
        if ctx.engine_handle is not None:
            names, dims = self._engine_names_dims()
            return EmbeddingBagCollectionAwaitable(awaitables=[NoWait(output[0])], embedding_dims=dims, embedding_names=names,
                                                   module_fqn=self._module_fqn, sharding_types=None)
        if not self._output_dists:
            self._create_output_dist()
        awaitables = [d(embs, sctx) for d, sctx, embs in zip(self._output_dists, ctx.sharding_contexts, output)]
        return self._finish_output(ctx, awaitables)

    def compute_and_output_dist(self, ctx: EmbeddingBagCollectionContext, input: KJTList) -> LazyAwaitable[KeyedTensor]:
        if isinstance(input, EngineDistInput):
            return self._engine_output(ctx)
        if not self._output_dists:
            self._create_output_dist()
        awaitables = []
        for lookup, d, sctx, features, sharding_type in zip(self._lookups, self._output_dists, ctx.sharding_contexts, input, self._sharding_types):
            with maybe_annotate_embedding_event(EmbeddingEvent.LOOKUP, self._module_fqn, sharding_type):
                embs = lookup(features)
            with maybe_annotate_embedding_event(EmbeddingEvent.OUTPUT_DIST, self._module_fqn, sharding_type):
                awaitables.append(d(embs, sctx))
            if self.post_lookup_tracker_fn is not None:
                self.post_lookup_tracker_fn(features, embs, self, None)
        return self._finish_output(ctx, awaitables)

    def _finish_output(self, ctx: EmbeddingBagCollectionContext, awaitables: List[Awaitable[torch.Tensor]]) -> LazyAwaitable[KeyedTensor]:
        if ctx.variable_batch_per_feature:
            assert ctx.inverse_indices is not None, "inverse indices must be provided from KJT if using variable batch size per feature."
            return VariableBatchEmbeddingBagCollectionAwaitable(
                awaitables=awaitables, inverse_indices=ctx.inverse_indices,
                inverse_indices_permute_indices=self._inverse_indices_permute_indices,
                batch_size_per_feature_pre_a2a=[b for s in ctx.sharding_contexts for b in s.batch_size_per_feature_pre_a2a],
                uncombined_embedding_dims=self._uncombined_embedding_dims, embedding_names=self._embedding_names,
                embedding_dims=self._embedding_dims, permute_op=self._permute_op,
            )
        awaitable = EmbeddingBagCollectionAwaitable(
            awaitables=awaitables, embedding_dims=self._pre_permute_dims(), embedding_names=self._pre_permute_names(),
            module_fqn=self._module_fqn, sharding_types=self._sharding_types,
        )
        if self._permute_op is not None:
            permute_op, names, dims = self._permute_op, self._embedding_names, self._embedding_dims

            def to_module_order(kt: KeyedTensor) -> KeyedTensor:
                return KeyedTensor(keys=names, length_per_key=dims, values=permute_op(kt.values()), key_dim=1)

            awaitable.callbacks.append(to_module_order)
        if self._has_mean_pooling_callback and ctx.divisor is not None:
            divisor = ctx.divisor
            awaitable.callbacks.append(lambda kt: _apply_mean_pooling(kt, divisor))
        return awaitable

    def _pre_permute_names(self) -> List[str]:
        if self._permute_op is None:
            return self._embedding_names
        return [n for s in self._embedding_shardings for n in s.embedding_names()]

    def _pre_permute_dims(self) -> List[int]:
        if self._permute_op is None:
            return self._embedding_dims
        return [d for s in self._embedding_shardings for d in s.embedding_dims()]


class EngineDistInput(Multistreamable):
    """What ``input_dist`` hands to ``compute`` when the fused sparse engine took the batch: the ids already sit in this
    rank's receive buffers; the handle names them."""

    def __init__(self, handle) -> None:
        self.handle = handle

    def record_stream(self, stream: torch.Stream) -> None:
        self.handle.record_stream(stream)


class _ViewParameter(nn.Parameter):
    """Parameter object sharing storage with a TBE table view; it never receives an autograd gradient
    (the kernel updates the table in backward) but keeps ``requires_grad`` semantics out of DDP's way."""

    def __new__(cls, data: torch.Tensor):
        return torch.Tensor._make_subclass(cls, data.detach(), False)


def _embedding_names_by_table(tables) -> List[List[str]]:
    shared: Dict[str, bool] = {}
    for cfg in tables:
        for f in cfg.feature_names:
            shared[f] = f in shared
    return [[f + "@" + cfg.name if shared[f] else f for f in cfg.feature_names] for cfg in tables]


def create_sharding_infos_by_sharding_device_group(module, table_name_to_parameter_sharding: Dict[str, ParameterSharding], prefix: str,
                                                   fused_params: Optional[Dict[str, Any]], suffix: Optional[str] = "weight",
                                                   ) -> Dict[Tuple[str, Any], List[EmbeddingShardingInfo]]:
    """The sharding infos of a collection keyed by (sharding type, device kind of the table's shards): a plan may keep some tables
    on GPUs and some in host memory, and each (type, kind) pair gets its own sharding object.
    (``torchrec/distributed/embeddingbag.py:185-280``.)"""
    from torchrec_b200.distributed.quant_input_dist import get_device_from_parameter_sharding

    by_type = ShardedEmbeddingBagCollection.create_grouped_sharding_infos(module, table_name_to_parameter_sharding, prefix, fused_params, suffix)
    out: Dict[Tuple[str, Any], List[EmbeddingShardingInfo]] = defaultdict(list)
    for sharding_type, infos in by_type.items():
        for info in infos:
            out[(sharding_type, get_device_from_parameter_sharding(info.param_sharding))].append(info)
    return dict(out)


class EmbeddingAwaitable(LazyAwaitable[torch.Tensor]):
    """The output of a sharded ``nn.EmbeddingBag``: the pooled rows once the exchange finished."""

    def __init__(self, awaitable: Awaitable[torch.Tensor]) -> None:
        super().__init__()
        self._awaitable = awaitable

    def _wait_impl(self) -> torch.Tensor:
        return self._awaitable.wait()


class ShardedEmbeddingBag(ShardedEmbeddingModule[KeyedJaggedTensor, torch.Tensor, torch.Tensor, NullShardedModuleContext], FusedOptimizerModule):
    """A single ``nn.EmbeddingBag`` (sum pooling) sharded row-wise, column-wise or data-parallel
    (``torchrec/distributed/embeddingbag.py:2013-2227``).  It is a one-table sharded collection under the hood: the bag's
    ``(input, offsets, per_sample_weights)`` call becomes a one-feature weighted KJT, and state-dict / parameter names lose the
    table prefix so that they read ``weight`` like the module it replaces."""

    _TABLE, _FEATURE = "embedding_bag", "ids"

    def __init__(self, module: nn.EmbeddingBag, table_name_to_parameter_sharding: Dict[str, ParameterSharding], env: ShardingEnv,
                 fused_params: Optional[Dict[str, Any]] = None, device: Optional[torch.device] = None) -> None:
        super().__init__()
        if len(table_name_to_parameter_sharding) != 1:
            raise AssertionError(f"expect 1 table, but got {len(table_name_to_parameter_sharding)}")
        if module.mode != "sum":
            raise AssertionError("ShardedEmbeddingBag only supports sum pooling")
        self.parameter_sharding: ParameterSharding = next(iter(table_name_to_parameter_sharding.values()))
        if self.parameter_sharding.sharding_type == ShardingType.TABLE_WISE.value:
            raise RuntimeError("table-wise sharding on a single EmbeddingBag is not supported yet")
        table = EmbeddingTableConfig(num_embeddings=module.num_embeddings, embedding_dim=module.embedding_dim, name=self._TABLE,
                                     feature_names=[self._FEATURE], pooling=PoolingType.SUM, is_weighted=True, embedding_names=[self._FEATURE])
        # the optimizer attached to the bag's weight (apply_optimizer_in_backward) becomes the kernel's in-backward optimizer
        per_table = ShardedEmbeddingBagCollection._table_fused_params(module.weight, self.parameter_sharding, fused_params or {})
        info = EmbeddingShardingInfo(embedding_config=table, param_sharding=self.parameter_sharding, param=module.weight, fused_params=per_table)
        self._env = env
        self._embedding_sharding = create_embedding_bag_sharding([info], env, device, permute_embeddings=True)
        self._input_dist: nn.Module = self._embedding_sharding.create_input_dist()
        self._lookup: nn.Module = self._embedding_sharding.create_lookup()
        self._output_dist: nn.Module = self._embedding_sharding.create_output_dist(device=device)
        found = []
        for kernel in self._lookup.modules():
            if isinstance(kernel, FusedOptimizerModule):
                kernel.fused_optimizer.params = {self._short(k): w for k, w in kernel.fused_optimizer.params.items()}
                found.append(("", kernel.fused_optimizer))
        self._optim: CombinedOptimizer = CombinedOptimizer(found)

    @staticmethod
    def _short(name: str) -> str:
        return name.rsplit(".", 1)[-1]

    # ---- stages ---------------------------------------------------------------------------------------------
    def create_context(self) -> NullShardedModuleContext:
        return NullShardedModuleContext()

    def input_dist(self, ctx: NullShardedModuleContext, input: torch.Tensor, offsets: Optional[torch.Tensor] = None,
                   per_sample_weights: Optional[torch.Tensor] = None) -> Awaitable[Awaitable[KeyedJaggedTensor]]:
        if offsets is None:  # 2-D input: every row is one bag
            assert input.dim() == 2, "offsets are required for 1-D input"
            offsets = torch.arange(0, input.numel() + 1, input.shape[1], device=input.device)
            input = input.reshape(-1)
        elif offsets.numel() == 0 or int(offsets[-1]) != input.numel():
            offsets = torch.cat([offsets, offsets.new_tensor([input.numel()])])  # nn.EmbeddingBag's offsets omit the end
        weights = per_sample_weights if per_sample_weights is not None else torch.ones_like(input, dtype=torch.float)
        features = KeyedJaggedTensor(keys=[self._FEATURE], values=input, offsets=offsets, weights=weights.reshape(-1))
        copies = len(self._embedding_sharding.feature_names())  # column shards each want the ids
        if copies != 1:
            features = features.permute([0] * copies)
        return self._input_dist(features)

    def compute(self, ctx: NullShardedModuleContext, dist_input: KeyedJaggedTensor) -> torch.Tensor:
        return self._lookup(dist_input)

    def output_dist(self, ctx: NullShardedModuleContext, output: torch.Tensor) -> LazyAwaitable[torch.Tensor]:
        return self._output_dist(output)

    # ---- state under the names of the module it replaces --------------------------------------------------------------
    def _checkpoint_weight(self):
        """``weight`` as the checkpoint sees it: a ``ShardedTensor`` over the group whose local shards are views of the kernel's
        memory (built once; collective on first use), or the plain tensor without a process group."""
        if "_weight_view" not in self.__dict__:
            local = [(t, w) for emb in self._lookup.emb_modules for t, w in zip(emb.config.embedding_tables, emb.split_embedding_weights())]
            pg = self._env.process_group
            if pg is None or self.parameter_sharding.sharding_type == ShardingType.DATA_PARALLEL.value:
                self.__dict__["_weight_view"] = local[0][1]
            else:
                self.__dict__["_weight_view"] = get_state_dict([t for t, _ in local], [w for _, w in local], pg=pg)[f"{self._TABLE}.weight"]
        return self.__dict__["_weight_view"]

    def state_dict(self, destination: Optional[Dict[str, Any]] = None, prefix: str = "", keep_vars: bool = False) -> Dict[str, Any]:
        out = OrderedDict() if destination is None else destination
        out[prefix + "weight"] = self._checkpoint_weight()
        return out

    def load_state_dict(self, state_dict, strict: bool = True):  # type: ignore[override]
        from torchrec_b200.distributed.embedding_lookup import _copy_checkpoint_entry

        missing = [] if "weight" in state_dict else ["weight"]
        if not missing:
            _copy_checkpoint_entry(self._checkpoint_weight(), state_dict["weight"])
        return torch.nn.modules.module._IncompatibleKeys(missing_keys=missing, unexpected_keys=[k for k in state_dict if k != "weight"])

    def named_modules(self, memo=None, prefix: str = "", remove_duplicate: bool = True):
        yield prefix, self

    def named_parameters(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True) -> Iterator[Tuple[str, nn.Parameter]]:
        """This rank's shard of the table as ``weight`` (a view of the kernel's memory; fused kernels update it in backward)."""
        views = self.__dict__.setdefault("_weight_views", {})
        for _, w in self._lookup.named_parameters_by_table():
            if w.data_ptr() not in views:
                views[w.data_ptr()] = w if isinstance(w, nn.Parameter) else _ViewParameter(w)
            yield append_prefix(prefix, "weight"), views[w.data_ptr()]

    def named_buffers(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True) -> Iterator[Tuple[str, torch.Tensor]]:
        for name, b in self._lookup.named_buffers("", recurse):
            yield append_prefix(prefix, self._short(name)), b

    def sharded_parameter_names(self, prefix: str = "") -> Iterator[str]:
        if self.parameter_sharding.sharding_type != ShardingType.DATA_PARALLEL.value:
            for name, _ in self.named_parameters(prefix):
                yield name

    @property
    def fused_optimizer(self) -> KeyedOptimizer:
        return self._optim

    @property
    def unsharded_module_type(self) -> Type[nn.EmbeddingBag]:
        return nn.EmbeddingBag


class EmbeddingBagSharder(BaseEmbeddingSharder[nn.EmbeddingBag]):
    """Shards a plain ``nn.EmbeddingBag`` (``torchrec/distributed/embeddingbag.py:2230-2255``)."""

    def shard(self, module: nn.EmbeddingBag, params: Dict[str, ParameterSharding], env: ShardingEnv,
              device: Optional[torch.device] = None, module_fqn: Optional[str] = None) -> ShardedEmbeddingBag:
        return ShardedEmbeddingBag(module, params, env, self.fused_params, device)

    def shardable_parameters(self, module: nn.EmbeddingBag) -> Dict[str, nn.Parameter]:
        return dict(module.named_parameters())

    @property
    def module_type(self) -> Type[nn.EmbeddingBag]:
        return nn.EmbeddingBag


class EmbeddingBagCollectionSharder(BaseEmbeddingSharder[EmbeddingBagCollection]):
    """Shards an ``EmbeddingBagCollection`` according to a module sharding plan."""

    def shard(self, module: EmbeddingBagCollection, params: Dict[str, ParameterSharding], env: ShardingEnv,
              device: Optional[torch.device] = None, module_fqn: Optional[str] = None) -> ShardedEmbeddingBagCollection:
        return ShardedEmbeddingBagCollection(
            module=module, table_name_to_parameter_sharding=params, env=env, fused_params=self.fused_params, device=device,
            qcomm_codecs_registry=self.qcomm_codecs_registry, module_fqn=module_fqn,
        )

    def shardable_parameters(self, module: EmbeddingBagCollection) -> Dict[str, nn.Parameter]:
        return {name.split(".")[0]: param for name, param in module.embedding_bags.named_parameters()}

    @property
    def module_type(self) -> Type[EmbeddingBagCollection]:
        return EmbeddingBagCollection
