"""Sharded ``EmbeddingCollection`` (unpooled / sequence embeddings).

Input dist as for pooled tables (plus optional per-feature id de-duplication), lookup returns one row
per id, and the sequence all-to-all sends every row back to the rank and position that asked for it.
The result is ``Dict[feature, JaggedTensor]`` exactly like the unsharded module; column-wise shards of
a table are concatenated along the embedding dim.

Counterpart of ``torchrec/distributed/embedding.py`` (``ShardedEmbeddingCollection`` ``:397``, index
dedup ``:1329``, sharder ``:1675``).
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

from torchrec_b200.distributed.batched_embedding_kernel import TableBatchedEmbeddingSlice, get_state_dict
from torchrec_b200.distributed.embedding_sharding import EmbeddingSharding, EmbeddingShardingInfo, KJTListSplitsAwaitable
from torchrec_b200.distributed.embeddingbag import ShardedTableStateMixin
from torchrec_b200.distributed.embedding_types import BaseEmbeddingSharder, EmbeddingComputeKernel, KJTList, ShardedEmbeddingModule
from torchrec_b200.distributed.sharding.cw_sequence_sharding import CwSequenceEmbeddingSharding
from torchrec_b200.distributed.sharding.dp_sequence_sharding import DpSequenceEmbeddingSharding
from torchrec_b200.distributed.sharding.rw_sequence_sharding import RwSequenceEmbeddingSharding
from torchrec_b200.distributed.sharding.rw_sharding import RwSparseFeaturesDist
from torchrec_b200.distributed.sharding.sequence_sharding import SequenceShardingContext
from torchrec_b200.distributed.sharding.tw_sequence_sharding import TwSequenceEmbeddingSharding
from torchrec_b200.distributed.types import (
    Awaitable,
    EmbeddingModuleShardingPlan,
    LazyAwaitable,
    NoWait,
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
    merge_fused_params,
    optimizer_type_to_emb_opt_type,
)
from torchrec_b200.modules.embedding_configs import EmbeddingConfig, EmbeddingTableConfig, PoolingType
from torchrec_b200.modules.embedding_modules import EmbeddingCollection, EmbeddingCollectionInterface
from torchrec_b200.ops import sparse_ops as sops
from torchrec_b200.optim.fused import EmptyFusedOptimizer, FusedOptimizerModule
from torchrec_b200.optim.keyed import CombinedOptimizer, KeyedOptimizer
from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor
from torchrec_b200.streamable import Multistreamable

EC_INDEX_DEDUP: bool = False


def get_ec_index_dedup() -> bool:
    return EC_INDEX_DEDUP


def set_ec_index_dedup(val: bool) -> None:
    """De-duplicate ids per feature before the input dist (smaller all-to-alls for repeated ids)."""
    global EC_INDEX_DEDUP
    EC_INDEX_DEDUP = val


def create_embedding_sharding(sharding_type: str, sharding_infos: List[EmbeddingShardingInfo], env: ShardingEnv,
                              device: Optional[torch.device] = None, qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None):
    by_type = {
        ShardingType.TABLE_WISE.value: TwSequenceEmbeddingSharding,
        ShardingType.ROW_WISE.value: RwSequenceEmbeddingSharding,
        ShardingType.COLUMN_WISE.value: CwSequenceEmbeddingSharding,
    }
    if sharding_type == ShardingType.DATA_PARALLEL.value:  # replicated tables exchange nothing: no codecs
        return DpSequenceEmbeddingSharding(sharding_infos, env, device)
    if sharding_type not in by_type:
        raise ValueError(f"Sharding not supported {sharding_type}")
    return by_type[sharding_type](sharding_infos, env, device, qcomm_codecs_registry=qcomm_codecs_registry)


def construct_jagged_tensors(embeddings: torch.Tensor, features: KeyedJaggedTensor, embedding_names: List[str], need_indices: bool = False,
                             features_to_permute_indices: Optional[Dict[str, List[int]]] = None,
                             original_features: Optional[KeyedJaggedTensor] = None, reverse_indices: Optional[torch.Tensor] = None) -> Dict[str, JaggedTensor]:
    """Cut ``embeddings [sum L, D]`` (key-major like ``features``) into one ``JaggedTensor`` per embedding name;
    several entries with the same name are column shards and are concatenated along dim 1."""
    with record_function("## construct_jagged_tensors ##"):
        if original_features is not None:
            features = original_features
        if reverse_indices is not None:
            embeddings = torch.index_select(embeddings, 0, reverse_indices.to(torch.int64))
        ret: Dict[str, JaggedTensor] = {}
        lengths = features.lengths().view(-1, features.stride())
        length_per_key = features.length_per_key()
        values = features.values()
        lengths_tuple = torch.unbind(lengths, dim=0)
        embeddings_list = torch.split(embeddings, length_per_key, dim=0)
        values_list = torch.split(values, length_per_key) if need_indices else None
        key_indices: Dict[str, List[int]] = defaultdict(list)
        for i, key in enumerate(embedding_names):
            key_indices[key].append(i)
        for key, indices in key_indices.items():
            if features_to_permute_indices and key in features_to_permute_indices:
                perm = features_to_permute_indices[key]
                indices = [indices[p] for p in perm] if len(perm) == len(indices) else indices
            ret[key] = JaggedTensor(
                lengths=lengths_tuple[indices[0]],
                values=embeddings_list[indices[0]] if len(indices) == 1 else torch.cat([embeddings_list[i] for i in indices], dim=1),
                weights=values_list[indices[0]] if values_list is not None else None,
            )
        return ret


def create_sharding_infos_by_sharding_device_group(module, table_name_to_parameter_sharding: Dict[str, ParameterSharding],
                                                   fused_params: Optional[Dict[str, Any]]) -> Dict[Tuple[str, Any], List[EmbeddingShardingInfo]]:
    """The sharding infos of a sequence collection keyed by (sharding type, device kind of the table's shards)
    (``torchrec/distributed/embedding.py:169-262``)."""
    from torchrec_b200.distributed.quant_input_dist import get_device_from_parameter_sharding

    by_type = ShardedEmbeddingCollection.create_grouped_sharding_infos(module, table_name_to_parameter_sharding, fused_params)
    out: Dict[Tuple[str, Any], List[EmbeddingShardingInfo]] = {}
    for sharding_type, infos in by_type.items():
        for info in infos:
            out.setdefault((sharding_type, get_device_from_parameter_sharding(info.param_sharding)), []).append(info)
    return out


def pad_vbe_kjt_lengths(features: KeyedJaggedTensor) -> KeyedJaggedTensor:
    """A variable-batch KJT as a fixed-batch one: every key's lengths padded with empty bags up to the largest per-key batch size.
    Values are untouched (the added bags are empty).  ``torchrec/distributed/embedding.py:264-285``."""
    strides = features.stride_per_key()
    max_stride = max(strides)
    lengths = features.lengths()
    padded = torch.zeros(max_stride * len(strides), device=lengths.device, dtype=lengths.dtype)
    start = 0
    for i, stride in enumerate(strides):
        padded[i * max_stride: i * max_stride + stride] = lengths[start: start + stride]
        start += stride
    return KeyedJaggedTensor(keys=features.keys(), values=features.values(), weights=features.weights_or_none(), lengths=padded, stride=max_stride,
                             length_per_key=features.length_per_key())


class EmbeddingCollectionContext(Multistreamable):
    def __init__(self, sharding_contexts: Optional[List[SequenceShardingContext]] = None, input_features: Optional[List[KeyedJaggedTensor]] = None,
                 reverse_indices: Optional[List[torch.Tensor]] = None) -> None:
        super().__init__()
        self.sharding_contexts: List[SequenceShardingContext] = sharding_contexts or []
        self.input_features: List[KeyedJaggedTensor] = input_features or []
        self.reverse_indices: List[torch.Tensor] = reverse_indices or []
        self.engine_handle = None  # set when the fused sequence engine distributed this batch
        self.engine_features: Optional[KeyedJaggedTensor] = None

    def record_stream(self, stream: torch.Stream) -> None:
        for ctx in self.sharding_contexts:
            ctx.record_stream(stream)
        for f in self.input_features:
            f.record_stream(stream)
        for r in self.reverse_indices:
            if r.is_cuda:
                r.record_stream(stream)
        if self.engine_handle is not None:
            self.engine_handle.record_stream(stream)


class EmbeddingCollectionAwaitable(LazyAwaitable[Dict[str, JaggedTensor]]):
    def __init__(self, awaitables_per_sharding: List[Awaitable[torch.Tensor]], features_per_sharding: List[KeyedJaggedTensor],
                 embedding_names_per_sharding: List[List[str]], ctx: EmbeddingCollectionContext, need_indices: bool = False,
                 features_to_permute_indices: Optional[Dict[str, List[int]]] = None) -> None:
        super().__init__()
        self._awaitables_per_sharding = awaitables_per_sharding
        self._features_per_sharding = features_per_sharding
        self._need_indices = need_indices
        self._features_to_permute_indices = features_to_permute_indices
        self._embedding_names_per_sharding = embedding_names_per_sharding
        self._ctx = ctx

    def _wait_impl(self) -> Dict[str, JaggedTensor]:
        jt_dict: Dict[str, JaggedTensor] = {}
        for i, (w, features, embedding_names) in enumerate(zip(self._awaitables_per_sharding, self._features_per_sharding, self._embedding_names_per_sharding)):
            original_features = self._ctx.input_features[i] if i < len(self._ctx.input_features) else None
            reverse_indices = self._ctx.reverse_indices[i] if i < len(self._ctx.reverse_indices) else None
            jt_dict.update(
                construct_jagged_tensors(
                    embeddings=w.wait(), features=features, embedding_names=embedding_names, need_indices=self._need_indices,
                    features_to_permute_indices=self._features_to_permute_indices, original_features=original_features,
                    reverse_indices=reverse_indices,
                )
            )
        return jt_dict


def _dedup_indices(ctx: EmbeddingCollectionContext, features: KeyedJaggedTensor, hash_offsets: torch.Tensor) -> KeyedJaggedTensor:
    """Replace ``features`` by its per-feature unique ids (one id per bag, lengths all 1 where kept) and
    remember in ``ctx`` how to expand looked-up rows back: rows for the original ids are
    ``unique_rows[reverse_indices]``.  Ids of different features never merge (offset by ``hash_offsets``)."""
    with record_function("## dedup_ec_indices ##"):
        values = features.values()
        counts, unique_ids, reverse = sops.unique_ids_per_feature(hash_offsets[: len(features.keys())], features.offsets(), values, bound=hash_offsets)
        stride = features.stride()
        # spread each feature's unique ids over its `stride` bags: first bags get ceil, rest floor (any split works,
        # the rows are re-expanded by `reverse` and the original lengths afterwards)
        base = torch.div(counts, stride, rounding_mode="floor")
        rem = counts - base * stride
        ar = torch.arange(stride, device=values.device)
        lengths = (base.unsqueeze(1) + (ar.unsqueeze(0) < rem.unsqueeze(1)).to(base.dtype)).reshape(-1)
        ctx.input_features.append(features)
        ctx.reverse_indices.append(reverse)
        return KeyedJaggedTensor(
            keys=features.keys(), values=unique_ids, lengths=lengths.to(features.lengths().dtype),
            stride=stride,
        )


class ShardedEmbeddingCollection(
    ShardedTableStateMixin,
    ShardedEmbeddingModule[KJTList, List[torch.Tensor], Dict[str, JaggedTensor], EmbeddingCollectionContext],
    FusedOptimizerModule,
):
    """Sharded counterpart of ``EmbeddingCollection``; built by ``EmbeddingCollectionSharder``.
    Table-wise, row-wise, column-wise and data-parallel placements (``torchrec/distributed/embedding.py:397``)."""

    _TABLE_ATTR: str = "embeddings"

    def _table_configs(self):
        return self._embedding_configs

    def __init__(self, module: EmbeddingCollection, table_name_to_parameter_sharding: Dict[str, ParameterSharding], env: ShardingEnv,
                 fused_params: Optional[Dict[str, Any]] = None, device: Optional[torch.device] = None,
                 qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None, use_index_dedup: bool = False,
                 module_fqn: Optional[str] = None) -> None:
        super().__init__(qcomm_codecs_registry=qcomm_codecs_registry)
        self._module_fqn = module_fqn
        self._embedding_configs: List[EmbeddingConfig] = module.embedding_configs()
        self._table_names: List[str] = [c.name for c in self._embedding_configs]
        self._table_name_to_config: Dict[str, EmbeddingConfig] = {c.name: c for c in self._embedding_configs}
        self.module_sharding_plan: EmbeddingModuleShardingPlan = EmbeddingModuleShardingPlan(
            {t: ps for t, ps in table_name_to_parameter_sharding.items() if t in self._table_names}
        )
        self._env = env
        self._device = device
        self._embedding_dim: int = module.embedding_dim()
        self._need_indices: bool = module.need_indices()
        self._use_index_dedup: bool = use_index_dedup or get_ec_index_dedup()
        self.sharding_type_to_sharding_infos = self.create_grouped_sharding_infos(module, table_name_to_parameter_sharding, fused_params)
        self._sharding_types: List[str] = list(self.sharding_type_to_sharding_infos.keys())
        self._embedding_shardings = [
            create_embedding_sharding(st, infos, env, device, qcomm_codecs_registry=self.qcomm_codecs_registry)
            for st, infos in self.sharding_type_to_sharding_infos.items()
        ]
        self._sharding_type_to_sharding = dict(zip(self._sharding_types, self._embedding_shardings))
        self._input_dists: List[nn.Module] = []
        self._lookups: List[nn.Module] = [s.create_lookup() for s in self._embedding_shardings]
        self._output_dists: List[nn.Module] = [s.create_output_dist() for s in self._embedding_shardings]
        self._feature_splits: List[int] = []
        self._features_order: List[int] = []
        self._has_uninitialized_input_dist: bool = True
        self._has_features_permute: bool = True
        self._embedding_names_per_sharding: List[List[str]] = [s.embedding_names() for s in self._embedding_shardings]
        self._features_to_permute_indices: Dict[str, List[int]] = self._column_shard_order()
        self._replicate_data_parallel_lookups(DpSequenceEmbeddingSharding)
        # parameters / ShardedTensor state: same layout logic as the pooled module, under "embeddings."
        self._output_dtensor = getattr(env, "output_dtensor", False)
        self._initialize_torch_state()
        self._optim: CombinedOptimizer = self._gather_fused_optimizers()
        self._hash_offsets_per_sharding: List[Optional[torch.Tensor]] = []
        self._engine = None
        self._engine_state: str = "auto"  # "auto" -> "on" | "off"

    # ---- plan -> sharding infos ---------------------------------------------------------------------
    @classmethod
    def create_grouped_sharding_infos(cls, module: EmbeddingCollection, table_name_to_parameter_sharding: Dict[str, ParameterSharding],
                                      fused_params: Optional[Dict[str, Any]]) -> Dict[str, List[EmbeddingShardingInfo]]:
        fused_params = fused_params or {}
        shared_feature: Dict[str, bool] = {}
        for cfg in module.embedding_configs():
            if not cfg.feature_names:
                cfg.feature_names = [cfg.name]
            for f in cfg.feature_names:
                shared_feature[f] = f in shared_feature
        out: Dict[str, List[EmbeddingShardingInfo]] = defaultdict(list)
        parameter_by_name = dict(module.named_parameters())
        state_dict = module.state_dict()
        for config in module.embedding_configs():
            table_name = config.name
            assert table_name in table_name_to_parameter_sharding, f"{table_name} not in table_name_to_parameter_sharding"
            ps = table_name_to_parameter_sharding[table_name]
            if ps.compute_kernel not in [k.value for k in EmbeddingComputeKernel]:
                raise ValueError(f"Compute kernel not supported {ps.compute_kernel}")
            param_name = "embeddings." + table_name + ".weight"
            assert param_name in parameter_by_name or param_name in state_dict
            param = parameter_by_name.get(param_name, state_dict.get(param_name))
            optimizer_params = getattr(param, "_optimizer_kwargs", [{}])
            optimizer_classes = getattr(param, "_optimizer_classes", [None])
            assert len(optimizer_classes) == 1 and len(optimizer_params) == 1, "Only support 1 optimizer per table"
            optimizer_params = copy.deepcopy(optimizer_params[0])
            if optimizer_classes[0]:
                optimizer_params["optimizer"] = optimizer_type_to_emb_opt_type(optimizer_classes[0])
            per_table = convert_to_fbgemm_types(add_params_from_parameter_sharding(merge_fused_params(fused_params, optimizer_params), ps))
            out[ps.sharding_type].append(
                EmbeddingShardingInfo(
                    embedding_config=EmbeddingTableConfig(
                        num_embeddings=config.num_embeddings, embedding_dim=config.embedding_dim, name=config.name,
                        data_type=config.data_type, feature_names=copy.deepcopy(config.feature_names), pooling=PoolingType.NONE,
                        is_weighted=False, has_feature_processor=False,
                        embedding_names=[f + "@" + config.name if shared_feature[f] else f for f in config.feature_names],
                        weight_init_max=config.weight_init_max, weight_init_min=config.weight_init_min, init_fn=config.init_fn,
                        total_num_buckets=getattr(config, "total_num_buckets", None),
                        use_virtual_table=getattr(config, "use_virtual_table", False),
                    ),
                    param_sharding=ps, param=param, fused_params=per_table,
                )
            )
        return out

    def _column_shard_order(self) -> Dict[str, List[int]]:
        """For every embedding name split column-wise: the order in which its pieces (as they appear in the
        sharding's embedding names, i.e. by rank) must be concatenated to restore ascending columns."""
        out: Dict[str, List[int]] = {}
        sharding = self._sharding_type_to_sharding.get(ShardingType.COLUMN_WISE.value)
        if sharding is None:
            return out
        col_offsets: Dict[str, List[int]] = defaultdict(list)
        for table in sharding.embedding_tables():
            off = table.local_metadata.shard_offsets[1] if table.local_metadata is not None else 0
            for name in table.embedding_names:
                col_offsets[name].append(off)
        for name, offs in col_offsets.items():
            order = sorted(range(len(offs)), key=lambda i: offs[i])
            if order != list(range(len(offs))):
                out[name] = order
        return out

    # ---- parameters / optimizer ---------------------------------------------------------------------
    def reset_parameters(self) -> None:
        return

    def named_parameters(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True) -> Iterator[Tuple[str, nn.Parameter]]:
        for name, m in self.embeddings.items():
            yield append_prefix(prefix, f"embeddings.{name}.weight"), m.weight

    def sharded_parameter_names(self, prefix: str = "") -> Iterator[str]:
        for name in self._model_parallel_name_to_local_shards.keys():
            yield append_prefix(prefix, f"embeddings.{name}.weight")

    @property
    def fused_optimizer(self) -> KeyedOptimizer:
        return self._optim

    @property
    def shardings(self) -> Dict[str, EmbeddingSharding]:
        return dict(zip(self._sharding_types, self._embedding_shardings))

    @property
    def unsharded_module_type(self) -> Type[EmbeddingCollection]:
        return EmbeddingCollection

    def create_context(self) -> EmbeddingCollectionContext:
        return EmbeddingCollectionContext(sharding_contexts=[])

    # ---- fused sequence engine ----------------------------------------------------------------------
    def disable_fused_engine(self) -> None:
        """Wrappers that change the distributed ids between input dist and lookup (managed collision) need the classic
        three-stage path."""
        self._engine_state, self._engine = "off", None

    def _fused_engine(self):
        if self._engine_state == "auto":
            self._engine = self._build_fused_engine()
            self._engine_state = "on" if self._engine is not None else "off"
        return self._engine

    def _build_fused_engine(self):
        """All ranks take the same decision: it depends on the plan, the environment and one collective agreement."""
        from torchrec_b200.distributed.fbgemm_qcomm_codec import CastCodec
        from torchrec_b200.distributed.fused_sequence_engine import FusedSequenceEngine
        from torchrec_b200.distributed.peer_memory import PeerGroup
        from torchrec_b200.distributed.types import CommOp

        dev = self._device
        if dev is None or dev.type != "cuda" or isinstance(self._env, ShardingEnv2D) or self._use_index_dedup:
            return None
        allowed = {ShardingType.TABLE_WISE.value, ShardingType.COLUMN_WISE.value, ShardingType.ROW_WISE.value}
        if not self._sharding_types or any(t not in allowed for t in self._sharding_types):
            return None
        fused = (EmbeddingComputeKernel.FUSED, EmbeddingComputeKernel.FUSED_UVM, EmbeddingComputeKernel.FUSED_UVM_CACHING)
        out_dtypes = set()
        for sh, lk in zip(self._embedding_shardings, self._lookups):
            if isinstance(lk, DistributedDataParallel):
                return None
            for groups in sh._grouped_embedding_configs_per_rank:
                if any(g.compute_kernel not in fused or g.has_feature_processor for g in groups):
                    return None
            for emb in lk.emb_modules:
                out_dtypes.add(emb.emb_module.output_dtype)
        if len(out_dtypes) > 1:
            return None
        out_dtype = out_dtypes.pop() if out_dtypes else torch.float32
        stage_dtype, grad_dtype = out_dtype, out_dtype
        codecs = (self.qcomm_codecs_registry or {}).get(CommOp.SEQUENCE_EMBEDDINGS_ALL_TO_ALL.name)
        if codecs is not None:
            fwd, bwd = codecs.forward, codecs.backward
            stage_dtype = fwd.quantized_dtype if isinstance(fwd, CastCodec) else torch.float16
            grad_dtype = bwd.quantized_dtype if isinstance(bwd, CastCodec) else torch.bfloat16
        peer = PeerGroup.get(self._env.process_group, dev)
        if peer is None:
            return None
        try:
            return FusedSequenceEngine(peer, self._embedding_configs, self._embedding_shardings, self._lookups, out_dtype, stage_dtype, grad_dtype)
        except AssertionError as e:
            import warnings

            warnings.warn(f"fused sequence engine not used for this module: {e}")
            return None

    def _engine_output(self, ctx: EmbeddingCollectionContext, rows: torch.Tensor) -> LazyAwaitable[Dict[str, JaggedTensor]]:
        """``rows [n, D]`` are in the order of the input KJT's values: cut them by that KJT's own lengths."""
        feats = ctx.engine_features
        wanted = self._engine.slot_names
        per_key = construct_jagged_tensors(rows, feats, list(feats.keys()), need_indices=self._need_indices)
        return NoWait({k: per_key[k] for k in wanted})

    # ---- the three stages ---------------------------------------------------------------------------
    def _create_input_dist(self, input_feature_names: List[str]) -> None:
        feature_names: List[str] = []
        for sharding in self._embedding_shardings:
            self._input_dists.append(sharding.create_input_dist())
            feature_names.extend(sharding.feature_names())
            self._feature_splits.append(len(sharding.feature_names()))
            hash_sizes = [0]
            for t in sharding.embedding_tables():
                for _ in t.feature_names:
                    hash_sizes.append(hash_sizes[-1] + t.num_embeddings)
            dev = self._device if self._device is not None and self._device.type != "meta" else torch.device("cpu")
            self._hash_offsets_per_sharding.append(torch.tensor(hash_sizes, dtype=torch.int64, device=dev))
        if feature_names == input_feature_names:
            self._has_features_permute = False
        else:
            self._features_order = [input_feature_names.index(f) for f in feature_names]
            dev = self._device if self._device is not None and self._device.type != "meta" else torch.device("cpu")
            self.register_buffer("_features_order_tensor", torch.tensor(self._features_order, device=dev, dtype=torch.int32), persistent=False)

    def input_dist(self, ctx: EmbeddingCollectionContext, features: KeyedJaggedTensor) -> Awaitable[Awaitable[KJTList]]:
        assert not features.variable_stride_per_key(), "variable batch per feature is not supported for sequence embeddings"
        engine = self._fused_engine() if self._engine_state != "off" else None
        if engine is not None and engine.accepts(features):
            from torchrec_b200.distributed.embeddingbag import EngineDistInput

            ctx.engine_handle = engine.input_dist(features)
            ctx.engine_features = features
            return NoWait(NoWait(EngineDistInput(ctx.engine_handle)))
        if self._has_uninitialized_input_dist:
            self._create_input_dist(features.keys())
            self._has_uninitialized_input_dist = False
        with torch.no_grad():
            if self._has_features_permute:
                features = features.permute(self._features_order, self._features_order_tensor)
            features_by_shards = features.split(self._feature_splits)
            awaitables = []
            for i, (input_dist, feats) in enumerate(zip(self._input_dists, features_by_shards)):
                if self._use_index_dedup and feats.values().numel() > 0:
                    feats = _dedup_indices(ctx, feats, self._hash_offsets_per_sharding[i])
                elif self._use_index_dedup:
                    ctx.input_features.append(feats)
                    ctx.reverse_indices.append(torch.empty(0, dtype=torch.int64, device=feats.values().device))
                awaitables.append(input_dist(feats))
                ctx.sharding_contexts.append(
                    SequenceShardingContext(
                        features_before_input_dist=feats,
                        unbucketize_permute_tensor=input_dist.unbucketize_permute_tensor if isinstance(input_dist, RwSparseFeaturesDist) else None,
                    )
                )
            return KJTListSplitsAwaitable(awaitables, ctx, self._module_fqn, self._sharding_types)

    def compute(self, ctx: EmbeddingCollectionContext, dist_input: KJTList) -> List[torch.Tensor]:
        if ctx.engine_handle is not None:
            return [self._engine.lookup(ctx.engine_handle)]
        ret: List[torch.Tensor] = []
        for lookup, features, sctx, sharding in zip(self._lookups, dist_input, ctx.sharding_contexts, self._embedding_shardings):
            sctx.lengths_after_input_dist = features.lengths().view(-1, features.stride())
            embs = lookup(features)
            if embs.dim() == 1:  # this rank holds no table of the sharding: keep the row width for the all-to-all
                # (requires_grad so that this rank still takes part in the backward all-to-all)
                embs = torch.empty((0, sharding.embedding_dims()[0]), dtype=embs.dtype, device=embs.device, requires_grad=True)
            ret.append(embs)
        return ret

    def output_dist(self, ctx: EmbeddingCollectionContext, output: List[torch.Tensor]) -> LazyAwaitable[Dict[str, JaggedTensor]]:
        if ctx.engine_handle is not None:
            return self._engine_output(ctx, output[0])
        awaitables: List[Awaitable[torch.Tensor]] = []
        features_before: List[KeyedJaggedTensor] = []
        for odist, embeddings, sctx in zip(self._output_dists, output, ctx.sharding_contexts):
            awaitables.append(odist(embeddings, sctx))
            features_before.append(sctx.features_before_input_dist)
        return EmbeddingCollectionAwaitable(
            awaitables_per_sharding=awaitables, features_per_sharding=features_before,
            embedding_names_per_sharding=self._embedding_names_per_sharding, need_indices=self._need_indices,
            features_to_permute_indices=self._features_to_permute_indices, ctx=ctx,
        )

    def compute_and_output_dist(self, ctx: EmbeddingCollectionContext, input: KJTList) -> LazyAwaitable[Dict[str, JaggedTensor]]:
        return self.output_dist(ctx, self.compute(ctx, input))

    # ---- embedding write path (``torchrec/distributed/embedding.py:1640-1672``) ----------------------------
    def write_dist(self, ctx: EmbeddingCollectionContext, embeddings: KeyedJaggedTensor) -> Awaitable[Awaitable[Any]]:
        """First half of an online row write: ``embeddings`` holds, per feature, the ids to overwrite (``values``) and the new
        rows (``weights``, ``[ids, D]``).  Every rank contributes its own writes; all of them reach every rank, and ``update``
        lets each rank keep what falls into its shards.  Writes are rare and small next to a training step, so they travel as
        one gather rather than through the sharding-specific id exchange."""
        rows = embeddings.weights()
        assert rows.dim() == 2 and rows.shape[0] == embeddings.values().numel(), "weights must hold one row per id"
        lpk = embeddings.length_per_key()
        mine = [(key, ids, r) for key, ids, r in zip(embeddings.keys(), embeddings.values().split(lpk), rows.split(lpk)) if ids.numel()]
        pg = self._env.process_group
        if pg is None or dist.get_world_size(pg) == 1:
            return NoWait(NoWait([mine]))
        gathered: List[Any] = [None] * dist.get_world_size(pg)
        dist.all_gather_object(gathered, [(k, i.cpu(), r.cpu()) for k, i, r in mine], group=pg)
        return NoWait(NoWait(gathered))

    @torch.no_grad()
    def update(self, ctx: EmbeddingCollectionContext, dist_input: Any) -> None:
        """Second half: write every received row (or its column slice) into the local shards whose row range holds the id.  Writes
        are applied in rank order, so on a conflict the highest rank's row stays, on every shard alike."""
        table_of = {f: cfg.name for cfg in self._embedding_configs for f in cfg.feature_names}
        for per_rank in dist_input:
            for feature, ids, rows in per_rank:
                table = table_of[feature]
                for _, lookup in self._unwrapped_lookups():
                    for emb in lookup.emb_modules:
                        for shard, weight in zip(emb.config.embedding_tables, emb.split_embedding_weights()):
                            if shard.name != table:
                                continue
                            (r0, c0), (nr, nc) = shard.local_metadata.shard_offsets, shard.local_metadata.shard_sizes
                            ids_d = ids.to(weight.device).long()
                            here = (ids_d >= r0) & (ids_d < r0 + nr)
                            if bool(here.any()):
                                weight[ids_d[here] - r0] = rows.to(weight.device)[here][:, c0: c0 + nc].to(weight.dtype)

    def write(self, embeddings: KeyedJaggedTensor) -> None:
        """``write_dist`` + ``update`` in one call (collective: every rank calls it, with an empty KJT if it has nothing to write)."""
        ctx = self.create_context()
        self.update(ctx, self.write_dist(ctx, embeddings).wait().wait())


class EmbeddingCollectionSharder(BaseEmbeddingSharder[EmbeddingCollection]):
    """Shards an ``EmbeddingCollection`` (``torchrec/distributed/embedding.py:1675``)."""

    def __init__(self, fused_params: Optional[Dict[str, Any]] = None, qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None,
                 use_index_dedup: bool = False) -> None:
        super().__init__(fused_params, qcomm_codecs_registry)
        self._use_index_dedup = use_index_dedup

    def shard(self, module: EmbeddingCollection, params: Dict[str, ParameterSharding], env: ShardingEnv,
              device: Optional[torch.device] = None, module_fqn: Optional[str] = None) -> ShardedEmbeddingCollection:
        return ShardedEmbeddingCollection(
            module, params, env, self.fused_params, device, qcomm_codecs_registry=self.qcomm_codecs_registry,
            use_index_dedup=self._use_index_dedup, module_fqn=module_fqn,
        )

    def shardable_parameters(self, module: EmbeddingCollection) -> Dict[str, nn.Parameter]:
        return {name.split(".")[0]: param for name, param in module.embeddings.named_parameters()}

    def sharding_types(self, compute_device_type: str) -> List[str]:
        return [ShardingType.DATA_PARALLEL.value, ShardingType.TABLE_WISE.value, ShardingType.COLUMN_WISE.value, ShardingType.ROW_WISE.value]

    @property
    def module_type(self) -> Type[EmbeddingCollection]:
        return EmbeddingCollection
