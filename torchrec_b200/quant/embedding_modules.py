"""Quantized (inference) ``EmbeddingBagCollection`` / ``EmbeddingCollection``.

Tables are stored row-wise quantized (int8 / int4 / int2, or fp16 / fp32) in the byte buffers of
``QuantTableBatchedEmbeddingBags``; tables that share pooling are batched into one lookup kernel.  ``from_float``
converts a trained module using each table's ``qconfig`` / ``data_type``; ``state_dict`` exposes the packed payload as
``embedding_bags.<t>.weight`` (uint8) and the row scales/biases as ``...weight_qscale`` / ``...weight_qbias`` views,
the same keys as ``torchrec/quant/embedding_modules.py:332-560`` (``quantize_state_dict`` ``:205``).
"""
from __future__ import annotations

import copy
from collections import OrderedDict, defaultdict
from typing import Any, Dict, List, Optional, Tuple

import torch
from torch import nn

from torchrec_b200.modules.embedding_configs import (
    DataType, EmbeddingBagConfig, EmbeddingConfig, PoolingType, QuantConfig, data_type_to_dtype, dtype_to_data_type, pooling_type_to_pooling_mode,
)
from torchrec_b200.modules.embedding_modules import (
    EmbeddingBagCollection as OriginalEmbeddingBagCollection,
    EmbeddingBagCollectionInterface,
    EmbeddingCollection as OriginalEmbeddingCollection,
    EmbeddingCollectionInterface,
    get_embedding_names_by_table,
)
from torchrec_b200.ops.qtbe import QuantTableBatchedEmbeddingBags
from torchrec_b200.ops.quant_ops import BITS, quantize_rowwise_nbit, row_bytes
from torchrec_b200.modules.embedding_configs import PoolingMode
from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor, KeyedTensor

MODULE_ATTR_REGISTER_TBES_BOOL: str = "__register_tbes_in_named_modules"
MODULE_ATTR_QUANT_STATE_DICT_SPLIT_SCALE_BIAS: str = "__quant_state_dict_split_scale_bias"
MODULE_ATTR_ROW_ALIGNMENT_INT: str = "__register_row_alignment_in_named_modules"
MODULE_ATTR_EMB_CONFIG_NAME_TO_NUM_ROWS_POST_PRUNING_DICT: str = "__emb_name_to_num_rows_post_pruning"
MODULE_ATTR_REMOVE_STBE_PADDING_BOOL: str = "__remove_stbe_padding"
MODULE_ATTR_USE_UNFLATTENED_LENGTHS_FOR_BATCHING: str = "__use_unflattened_lengths_for_batching"
MODULE_ATTR_USE_BATCHING_HINTED_OUTPUT: str = "__use_batching_hinted_output"
MODULE_ATTR_CACHE_FEATURES_ORDER: str = "__cache_features_order"
DEFAULT_ROW_ALIGNMENT = 16


# ---- marks that the float modules carry into ``from_float`` ----------------------------------------------------------------
# A conversion pass (``torch.quantization.convert`` style) reads these attributes from the float module it replaces; the helpers
# below set them on every submodule of the given types before the conversion runs.
def for_each_module_of_type_do(module: nn.Module, module_types: List[type], op) -> None:
    for m in module.modules():
        if isinstance(m, tuple(module_types)):
            op(m)


def _mark(module: nn.Module, module_types: List[type], attr: str, value) -> None:
    for_each_module_of_type_do(module, module_types, lambda m: setattr(m, attr, value))


def quant_prep_enable_quant_state_dict_split_scale_bias(module: nn.Module) -> None:
    """The quantized module's state dict lists every table's scale and bias columns as a tensor of their own."""
    setattr(module, MODULE_ATTR_QUANT_STATE_DICT_SPLIT_SCALE_BIAS, True)


def quant_prep_enable_quant_state_dict_split_scale_bias_for_types(module: nn.Module, module_types: List[type]) -> None:
    _mark(module, module_types, MODULE_ATTR_QUANT_STATE_DICT_SPLIT_SCALE_BIAS, True)


def quant_prep_enable_register_tbes(module: nn.Module, module_types: List[type]) -> None:
    """The quantized module registers its lookup kernels as submodules (visible to ``named_modules``)."""
    _mark(module, module_types, MODULE_ATTR_REGISTER_TBES_BOOL, True)


def quant_prep_customize_row_alignment(module: nn.Module, module_types: List[type], row_alignment: int) -> None:
    """Byte alignment of the quantized rows (the default is 16)."""
    _mark(module, module_types, MODULE_ATTR_ROW_ALIGNMENT_INT, row_alignment)


def quant_prep_enable_cache_features_order(module: nn.Module, module_types: List[type]) -> None:
    """The quantized module remembers the feature permutation of its first request instead of recomputing it per request."""
    _mark(module, module_types, MODULE_ATTR_CACHE_FEATURES_ORDER, True)


def quantize_state_dict(module: nn.Module, table_name_to_quantized_weights: Dict[str, Tuple[torch.Tensor, Optional[torch.Tensor]]],
                        table_name_to_data_type: Dict[str, DataType], table_name_to_num_embeddings_post_pruning: Optional[Dict[str, int]] = None) -> torch.device:
    """Quantize every ``embedding(_bag)s.<table>.weight`` of ``module``'s state dict row-wise to the table's data type.
    Fills ``table_name_to_quantized_weights[table] = (packed uint8 [R, row_bytes], None)`` and returns the weights' device."""
    device = torch.device("cpu")
    if not table_name_to_num_embeddings_post_pruning:
        table_name_to_num_embeddings_post_pruning = {}
    for key, tensor in module.state_dict().items():
        splits = key.split(".")
        assert splits[-1] == "weight"
        table_name = splits[-2]
        data_type = table_name_to_data_type[table_name]
        num_rows = tensor.shape[0]
        if table_name in table_name_to_num_embeddings_post_pruning:
            num_rows = table_name_to_num_embeddings_post_pruning[table_name]
        device = tensor.device
        if tensor.is_meta:
            bits = BITS[data_type]
            packed = torch.empty(num_rows, row_bytes(tensor.shape[1], bits), dtype=torch.uint8, device="meta")
        else:
            packed = quantize_rowwise_nbit(tensor[:num_rows].float(), BITS[data_type])
        table_name_to_quantized_weights[table_name] = (packed, None)
    return device


def _data_type_of(table, module_qconfig) -> DataType:
    """Target storage type: explicit per-table ``data_type`` if it is a quantized type, else from the module's qconfig."""
    if module_qconfig is not None:
        w = module_qconfig.weight() if callable(getattr(module_qconfig, "weight", None)) else None
        dt = getattr(w, "dtype", None)
        if dt is not None:
            return {torch.quint8: DataType.INT8, torch.qint8: DataType.INT8, torch.quint4x2: DataType.INT4, torch.quint2x4: DataType.INT2,
                    torch.float16: DataType.FP16, torch.float32: DataType.FP32}.get(dt, DataType.INT8)
    return table.data_type


class _QuantCollectionBase(nn.Module):
    """Shared storage logic: group tables, pack weights, state-dict views."""

    _container: str = "embedding_bags"

    def _build(self, tables, table_name_to_quantized_weights, device, output_dtype, pooled: bool, row_alignment: int) -> None:
        self._output_dtype = output_dtype
        self._device = device
        self._key_to_tables: Dict[Any, List[Any]] = defaultdict(list)
        for t in tables:
            key = (t.pooling if pooled else PoolingType.NONE)
            self._key_to_tables[key].append(t)
        self._emb_modules: nn.ModuleList = nn.ModuleList()
        self._group_tables: List[List[Any]] = []
        self._feature_splits: List[int] = []
        container = nn.ModuleDict()
        setattr(self, self._container, container)
        for key, group in self._key_to_tables.items():
            specs = [(t.num_embeddings_post_pruning or t.num_embeddings if hasattr(t, "num_embeddings_post_pruning") else t.num_embeddings, t.embedding_dim, BITS[t.data_type]) for t in group]
            ftm = [i for i, t in enumerate(group) for _ in t.feature_names]
            mode = pooling_type_to_pooling_mode(key) if pooled else PoolingMode.NONE
            emb = QuantTableBatchedEmbeddingBags(specs, ftm, mode, output_dtype, device=device, persistent_weights=False)
            for i, t in enumerate(group):
                if table_name_to_quantized_weights and t.name in table_name_to_quantized_weights:
                    packed = table_name_to_quantized_weights[t.name][0]
                    if not packed.is_meta:
                        emb.table_view(i).copy_(packed.to(emb.weights.device))
                holder = nn.Module()
                holder.register_buffer("weight", emb.table_view(i))
                container[t.name] = holder
            self._emb_modules.append(emb)
            self._group_tables.append(group)
            self._feature_splits.append(len(ftm))
        self._feature_names: List[str] = [f for group in self._group_tables for t in group for f in t.feature_names]

    def _packed_tables(self):
        """(table config, packed rows as stored by the kernel) for every table."""
        for group, emb in zip(self._group_tables, self._emb_modules):
            for i, t in enumerate(group):
                yield t, emb.table_view(i)

    def _split_scale_bias_state(self, destination: Dict[str, Any], prefix: str) -> None:
        for group, emb in zip(self._group_tables, self._emb_modules):
            for i, t in enumerate(group):
                bits = BITS[t.data_type]
                if bits >= 16:
                    continue
                view = emb.table_view(i)
                nb = t.embedding_dim * bits // 8
                sb = view[:, nb: nb + 4].contiguous().view(torch.float16).view(-1, 2)
                destination[f"{prefix}{self._container}.{t.name}.weight"] = view[:, :nb]
                destination[f"{prefix}{self._container}.{t.name}.weight_qscale"] = sb[:, 0]
                destination[f"{prefix}{self._container}.{t.name}.weight_qbias"] = sb[:, 1]

    def state_dict(self, *args, destination=None, prefix="", keep_vars=False):
        sd = super().state_dict(*args, destination=destination, prefix=prefix, keep_vars=keep_vars)
        if getattr(self, MODULE_ATTR_QUANT_STATE_DICT_SPLIT_SCALE_BIAS, False):
            self._split_scale_bias_state(sd, prefix)
        return sd

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        """Accept the split form (payload + ``_qscale`` / ``_qbias``): merge it back into packed rows before the per-table
        buffers load (this hook runs before the children's)."""
        for group, emb in zip(self._group_tables, self._emb_modules):
            for i, t in enumerate(group):
                k = f"{prefix}{self._container}.{t.name}.weight"
                qs, qb = state_dict.pop(k + "_qscale", None), state_dict.pop(k + "_qbias", None)
                if k in state_dict and qs is not None and qb is not None and state_dict[k].shape[1] != emb.table_view(i).shape[1]:
                    tail = torch.stack([qs.half(), qb.half()], 1).contiguous().view(torch.uint8).view(-1, 4)
                    state_dict[k] = torch.cat([state_dict[k], tail.to(state_dict[k].device)], dim=1)
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs)

    def tbes_in_named_modules(self) -> bool:
        return getattr(self, MODULE_ATTR_REGISTER_TBES_BOOL, False)

    @property
    def device(self) -> torch.device:
        return self._emb_modules[0].weights.device if len(self._emb_modules) else torch.device("cpu")


class EmbeddingBagCollection(EmbeddingBagCollectionInterface, _QuantCollectionBase):
    """Quantized pooled lookups: ``forward(KJT) -> KeyedTensor [B, sum D]``."""

    _container = "embedding_bags"

    def __init__(self, tables: List[EmbeddingBagConfig], is_weighted: bool, device: torch.device, output_dtype: torch.dtype = torch.float,
                 table_name_to_quantized_weights: Optional[Dict[str, Tuple[torch.Tensor, Optional[torch.Tensor]]]] = None,
                 register_tbes: bool = False, quant_state_dict_split_scale_bias: bool = False, row_alignment: int = DEFAULT_ROW_ALIGNMENT,
                 cache_features_order: bool = False) -> None:
        super().__init__()
        self._is_weighted = is_weighted
        self._embedding_bag_configs = tables
        names = set()
        for t in tables:
            if t.name in names:
                raise ValueError(f"Duplicate table name {t.name}")
            names.add(t.name)
        self._build(tables, table_name_to_quantized_weights, device, output_dtype, pooled=True, row_alignment=row_alignment)
        self._embedding_names: List[str] = [n for names_ in get_embedding_names_by_table(tables) for n in names_]
        self._length_per_key: List[int] = [t.embedding_dim for group in self._group_tables for t in group for _ in t.feature_names]
        # group order may differ from table order: map to the unsharded module's key order
        grouped_names = [n for group in self._group_tables for names_ in get_embedding_names_by_table(group) for n in names_]
        shared = dict(zip([f"{t.name}:{f}" for t in tables for f in t.feature_names], self._embedding_names))
        grouped_names = [shared[f"{t.name}:{f}"] for group in self._group_tables for t in group for f in t.feature_names]
        self._grouped_names: List[str] = grouped_names
        self._out_perm: Optional[List[int]] = None
        if grouped_names != self._embedding_names:
            self._out_perm = [grouped_names.index(n) for n in self._embedding_names]
        self._grouped_dims = list(self._length_per_key)
        self._length_per_key = [t.embedding_dim for t in tables for _ in t.feature_names]
        setattr(self, MODULE_ATTR_REGISTER_TBES_BOOL, register_tbes)
        setattr(self, MODULE_ATTR_QUANT_STATE_DICT_SPLIT_SCALE_BIAS, quant_state_dict_split_scale_bias)

    def forward(self, features: KeyedJaggedTensor) -> KeyedTensor:
        kjt = features.permute([features.keys().index(f) for f in self._feature_names]) if features.keys() != self._feature_names else features
        groups = kjt.split(self._feature_splits) if len(self._emb_modules) > 1 else [kjt]
        outs = []
        for emb, f in zip(self._emb_modules, groups):
            outs.append(emb(f.values(), f.offsets(), f.weights_or_none() if self._is_weighted else None))
        values = outs[0] if len(outs) == 1 else torch.cat(outs, dim=1)
        if self._out_perm is not None:
            pieces = values.split(self._grouped_dims, dim=1)
            values = torch.cat([pieces[i] for i in self._out_perm], dim=1)
        return KeyedTensor(keys=self._embedding_names, values=values, length_per_key=self._length_per_key)

    def forward_into(self, features: KeyedJaggedTensor, out: torch.Tensor, column_of: Dict[str, int]) -> None:
        """Pooled lookups stored straight into ``out [B, width]`` at ``column_of[embedding name]`` (a buffer that may belong to
        another device of this process): what a sharded serving model uses instead of returning pieces to be copied and joined."""
        kjt = features.permute([features.keys().index(f) for f in self._feature_names]) if features.keys() != self._feature_names else features
        groups = kjt.split(self._feature_splits) if len(self._emb_modules) > 1 else [kjt]
        names = iter(self._grouped_names)
        for emb, f in zip(self._emb_modules, groups):
            cols = [column_of[next(names)] for _ in emb.feature_table_map]
            emb.forward_into(f.values(), f.offsets(), f.weights_or_none() if self._is_weighted else None, out, cols)

    @classmethod
    def from_float(cls, module: OriginalEmbeddingBagCollection, use_precomputed_fake_quant: bool = False) -> "EmbeddingBagCollection":
        assert hasattr(module, "qconfig"), "EmbeddingBagCollection input float module must have qconfig defined"
        pruning = getattr(module, MODULE_ATTR_EMB_CONFIG_NAME_TO_NUM_ROWS_POST_PRUNING_DICT, {}) or {}
        tables = copy.deepcopy(module.embedding_bag_configs())
        data_type = _data_type_of(tables[0], module.qconfig) if tables else DataType.INT8
        per_table = getattr(module.qconfig, "per_table_weight_dtype", None) if isinstance(module.qconfig, QuantConfig) else None
        name_to_dt: Dict[str, DataType] = {}
        for t in tables:
            dt = data_type
            if per_table and t.name in per_table:
                dt = dtype_to_data_type(per_table[t.name])
            t.data_type = dt
            name_to_dt[t.name] = dt
            if t.name in pruning:
                t.num_embeddings_post_pruning = pruning[t.name]
        quantized: Dict[str, Tuple[torch.Tensor, Optional[torch.Tensor]]] = {}
        device = quantize_state_dict(module, quantized, name_to_dt, pruning)
        out_dtype = module.qconfig.activation().dtype if callable(getattr(module.qconfig, "activation", None)) else torch.float
        return cls(tables, module.is_weighted(), device=device, output_dtype=out_dtype if out_dtype in (torch.float, torch.half, torch.bfloat16) else torch.float,
                   table_name_to_quantized_weights=quantized, register_tbes=getattr(module, MODULE_ATTR_REGISTER_TBES_BOOL, False),
                   quant_state_dict_split_scale_bias=getattr(module, MODULE_ATTR_QUANT_STATE_DICT_SPLIT_SCALE_BIAS, False),
                   row_alignment=getattr(module, MODULE_ATTR_ROW_ALIGNMENT_INT, DEFAULT_ROW_ALIGNMENT))

    def embedding_bag_configs(self) -> List[EmbeddingBagConfig]:
        return self._embedding_bag_configs

    def is_weighted(self) -> bool:
        return self._is_weighted

    def output_dtype(self) -> torch.dtype:
        return self._output_dtype


class FeatureProcessedEmbeddingBagCollection(EmbeddingBagCollection):
    """Quantized pooled lookups behind feature processors (position weights and the like): the processors rewrite the per-id
    weights of the incoming KJT, the quantized kernel pools with them (``torchrec/quant/embedding_modules.py:633-731``)."""

    def __init__(self, tables: List[EmbeddingBagConfig], is_weighted: bool, device: torch.device, output_dtype: torch.dtype = torch.float,
                 table_name_to_quantized_weights: Optional[Dict[str, Tuple[torch.Tensor, Optional[torch.Tensor]]]] = None,
                 register_tbes: bool = False, quant_state_dict_split_scale_bias: bool = False, row_alignment: int = DEFAULT_ROW_ALIGNMENT,
                 feature_processor: Optional[nn.Module] = None, cache_features_order: bool = False) -> None:
        if feature_processor is None:
            raise AssertionError("Use EmbeddingBagCollection for no feature_processor")
        super().__init__(tables, is_weighted, device, output_dtype, table_name_to_quantized_weights, register_tbes,
                         quant_state_dict_split_scale_bias, row_alignment, cache_features_order)
        self.feature_processor = feature_processor

    def forward(self, features: KeyedJaggedTensor) -> KeyedTensor:
        return super().forward(self.feature_processor(features))

    def _get_name(self) -> str:
        return "QuantFeatureProcessedEmbeddingBagCollection"

    @classmethod
    def from_float(cls, module: nn.Module, use_precomputed_fake_quant: bool = False) -> "FeatureProcessedEmbeddingBagCollection":
        assert hasattr(module, "qconfig"), "FeatureProcessedEmbeddingBagCollection input float module must have qconfig defined"
        inner = module._embedding_bag_collection
        # the wrapped collection is converted by the plain class method, under the wrapper's settings
        for attr in ("qconfig", MODULE_ATTR_EMB_CONFIG_NAME_TO_NUM_ROWS_POST_PRUNING_DICT, MODULE_ATTR_REGISTER_TBES_BOOL):
            if hasattr(module, attr):
                setattr(inner, attr, getattr(module, attr))
        plain = EmbeddingBagCollection.from_float(inner)
        packed = {t.name: (w, None) for t, w in plain._packed_tables()}
        return cls(plain.embedding_bag_configs(), plain.is_weighted(), device=plain.device, output_dtype=plain.output_dtype(),
                   table_name_to_quantized_weights=packed, register_tbes=getattr(module, MODULE_ATTR_REGISTER_TBES_BOOL, False),
                   quant_state_dict_split_scale_bias=getattr(inner, MODULE_ATTR_QUANT_STATE_DICT_SPLIT_SCALE_BIAS, False),
                   row_alignment=getattr(inner, MODULE_ATTR_ROW_ALIGNMENT_INT, DEFAULT_ROW_ALIGNMENT),
                   feature_processor=module._feature_processors, cache_features_order=getattr(module, MODULE_ATTR_CACHE_FEATURES_ORDER, False))


class EmbeddingCollection(EmbeddingCollectionInterface, _QuantCollectionBase):
    """Quantized unpooled lookups: ``forward(KJT) -> Dict[feature, JaggedTensor]``."""

    _container = "embeddings"

    def __init__(self, tables: List[EmbeddingConfig], device: torch.device, need_indices: bool = False, output_dtype: torch.dtype = torch.float,
                 table_name_to_quantized_weights: Optional[Dict[str, Tuple[torch.Tensor, Optional[torch.Tensor]]]] = None,
                 register_tbes: bool = False, quant_state_dict_split_scale_bias: bool = False, row_alignment: int = DEFAULT_ROW_ALIGNMENT,
                 cache_features_order: bool = False) -> None:
        super().__init__()
        self._embedding_configs = tables
        self._need_indices = need_indices
        self._embedding_dim = tables[0].embedding_dim if tables else -1
        for t in tables:
            assert t.embedding_dim == self._embedding_dim, "All tables in a EmbeddingCollection are required to have same embedding dimension."
        self._build(tables, table_name_to_quantized_weights, device, output_dtype, pooled=False, row_alignment=row_alignment)
        self._embedding_names_by_table = get_embedding_names_by_table(tables)
        self._name_of: Dict[str, str] = {}
        for t, names_ in zip(tables, self._embedding_names_by_table):
            for f, n in zip(t.feature_names, names_):
                self._name_of[f"{t.name}:{f}"] = n
        setattr(self, MODULE_ATTR_REGISTER_TBES_BOOL, register_tbes)
        setattr(self, MODULE_ATTR_QUANT_STATE_DICT_SPLIT_SCALE_BIAS, quant_state_dict_split_scale_bias)

    def forward(self, features: KeyedJaggedTensor) -> Dict[str, JaggedTensor]:
        kjt = features.permute([features.keys().index(f) for f in self._feature_names]) if features.keys() != self._feature_names else features
        groups = kjt.split(self._feature_splits) if len(self._emb_modules) > 1 else [kjt]
        out: Dict[str, JaggedTensor] = {}
        for emb, f, group in zip(self._emb_modules, groups, self._group_tables):
            rows = emb(f.values(), f.offsets())
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

    @classmethod
    def from_float(cls, module: OriginalEmbeddingCollection, use_precomputed_fake_quant: bool = False) -> "EmbeddingCollection":
        assert hasattr(module, "qconfig"), "EmbeddingCollection input float module must have qconfig defined"
        tables = copy.deepcopy(module.embedding_configs())
        data_type = _data_type_of(tables[0], module.qconfig) if tables else DataType.INT8
        name_to_dt = {}
        for t in tables:
            t.data_type = data_type
            name_to_dt[t.name] = data_type
        quantized: Dict[str, Tuple[torch.Tensor, Optional[torch.Tensor]]] = {}
        device = quantize_state_dict(module, quantized, name_to_dt, None)
        return cls(tables, device=device, need_indices=module.need_indices(), table_name_to_quantized_weights=quantized,
                   register_tbes=getattr(module, MODULE_ATTR_REGISTER_TBES_BOOL, False),
                   quant_state_dict_split_scale_bias=getattr(module, MODULE_ATTR_QUANT_STATE_DICT_SPLIT_SCALE_BIAS, False))

    def embedding_configs(self) -> List[EmbeddingConfig]:
        return self._embedding_configs

    def embedding_dim(self) -> int:
        return self._embedding_dim

    def embedding_names_by_table(self) -> List[List[str]]:
        return self._embedding_names_by_table

    def need_indices(self) -> bool:
        return self._need_indices

    def output_dtype(self) -> torch.dtype:
        return self._output_dtype


class QuantManagedCollisionEmbeddingCollection(EmbeddingCollection):
    """Quantized unpooled lookups behind managed-collision modules: raw ids are first mapped to table slots by the trained id
    maps (serving never admits or evicts), then looked up.  ``forward`` returns ``(embeddings, remapped KJT)``
    (``torchrec/quant/embedding_modules.py:1029-1190``)."""

    def __init__(self, tables: List[EmbeddingConfig], device: torch.device, need_indices: bool = False, output_dtype: torch.dtype = torch.float,
                 table_name_to_quantized_weights: Optional[Dict[str, Tuple[torch.Tensor, Optional[torch.Tensor]]]] = None,
                 register_tbes: bool = False, quant_state_dict_split_scale_bias: bool = False, row_alignment: int = DEFAULT_ROW_ALIGNMENT,
                 managed_collision_collection: Optional[nn.Module] = None, return_remapped_features: bool = False,
                 cache_features_order: bool = False) -> None:
        if not managed_collision_collection:
            raise AssertionError("Managed collision collection cannot be None")
        super().__init__(tables, device, need_indices, output_dtype, table_name_to_quantized_weights, register_tbes,
                         quant_state_dict_split_scale_bias, row_alignment, cache_features_order)
        self._managed_collision_collection = managed_collision_collection
        self._return_remapped_features = return_remapped_features
        ours = [(t.name, t.num_embeddings, t.embedding_dim, tuple(t.feature_names)) for t in self.embedding_configs()]
        theirs = [(t.name, t.num_embeddings, t.embedding_dim, tuple(t.feature_names)) for t in managed_collision_collection.embedding_configs()]
        assert ours == theirs, "Embedding Collection and Managed Collision Collection must contain the same Embedding Configs"
        managed_collision_collection.eval()
        for mc in managed_collision_collection._managed_collision_modules.values():
            mc.reset_inference_mode()

    def forward(self, features: KeyedJaggedTensor):
        remapped = self._managed_collision_collection(features)
        return super().forward(remapped), remapped

    def _get_name(self) -> str:
        return "QuantManagedCollisionEmbeddingCollection"

    @classmethod
    def from_float(cls, module: nn.Module, return_remapped_features: bool = False) -> "QuantManagedCollisionEmbeddingCollection":
        assert hasattr(module, "qconfig"), "QuantManagedCollisionEmbeddingCollection input float module must have qconfig defined"
        inner = module._embedding_module
        if isinstance(inner, EmbeddingCollection):  # already quantized: take its packed tables as they are
            plain = inner
        else:
            inner.qconfig = module.qconfig
            plain = EmbeddingCollection.from_float(inner)
        mcc = module._managed_collision_collection
        for cfg, qcfg in zip(mcc.embedding_configs(), plain.embedding_configs()):
            cfg.data_type = qcfg.data_type
        packed = {t.name: (w, None) for t, w in plain._packed_tables()}
        return cls(plain.embedding_configs(), device=plain.device, need_indices=plain.need_indices(), output_dtype=plain.output_dtype(),
                   table_name_to_quantized_weights=packed, register_tbes=getattr(module, MODULE_ATTR_REGISTER_TBES_BOOL, False),
                   quant_state_dict_split_scale_bias=getattr(inner, MODULE_ATTR_QUANT_STATE_DICT_SPLIT_SCALE_BIAS, False),
                   row_alignment=getattr(inner, MODULE_ATTR_ROW_ALIGNMENT_INT, DEFAULT_ROW_ALIGNMENT), managed_collision_collection=mcc,
                   return_remapped_features=getattr(module, "_return_remapped_features", return_remapped_features),
                   cache_features_order=getattr(inner, MODULE_ATTR_CACHE_FEATURES_ORDER, False))
