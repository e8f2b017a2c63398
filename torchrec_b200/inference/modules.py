"""From a trained model to a served one: quantize the embeddings (and optionally the dense part), shard the quantized
tables over the devices of one host, wrap the result for a batching server.

    qmodel = quantize_inference_model(model)                  # EBC/EC -> row-wise int8/int4 modules
    smodel, plan = shard_quant_model(qmodel, world_size=N)    # table-wise placement on N devices, one process
    PredictFactory / PredictModule                            # packaging contract of the serving runtime

Counterpart of ``torchrec/inference/modules.py`` (``quantize_embeddings`` ``:139``, ``quantize_inference_model`` ``:376``,
``shard_quant_model`` ``:493``, ``PredictFactory`` ``:191``, ``PredictModule`` ``:268``).
"""
from __future__ import annotations

import abc
import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple, Type, Union

import torch
import torch.ao.quantization as tq
from torch import nn

from torchrec_b200.distributed.quant_embedding import QuantEmbeddingCollectionSharder, ShardedQuantEmbeddingCollection
from torchrec_b200.distributed.quant_embeddingbag import QuantEmbeddingBagCollectionSharder, ShardedQuantEmbeddingBagCollection
from torchrec_b200.distributed.types import ParameterSharding, ShardingEnv, ShardingPlan, ShardingType
from torchrec_b200.modules.embedding_configs import DataType, QuantConfig, data_type_to_dtype
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection, EmbeddingCollection
from torchrec_b200.quant.embedding_modules import (
    MODULE_ATTR_EMB_CONFIG_NAME_TO_NUM_ROWS_POST_PRUNING_DICT,
    EmbeddingBagCollection as QuantEmbeddingBagCollection,
    EmbeddingCollection as QuantEmbeddingCollection,
    quant_prep_enable_quant_state_dict_split_scale_bias,
    quant_prep_enable_register_tbes,
)

DEFAULT_FUSED_PARAMS: Dict[str, Any] = {
    "__register_quant_state_dict_split_scale_bias": True,
    "__register_row_alignment_in_named_modules": 16,
    "__emb_name_to_num_rows_post_pruning": {},
}
DEFAULT_SHARDERS = [QuantEmbeddingBagCollectionSharder(), QuantEmbeddingCollectionSharder()]
DEFAULT_QUANT_MAPPING: Dict[str, Type[nn.Module]] = {
    "torchrec_b200.modules.embedding_modules.EmbeddingBagCollection": QuantEmbeddingBagCollection,
    "torchrec_b200.modules.embedding_modules.EmbeddingCollection": QuantEmbeddingCollection,
}
DEFAULT_QUANTIZATION_DTYPE: torch.dtype = torch.int8


def trim_torch_package_prefix_from_typename(typename: str) -> str:
    if typename.startswith("<torch_package_"):
        typename = ".".join(typename.split(".")[1:])
    return typename


def _qdtype(dtype: torch.dtype) -> torch.dtype:
    return {torch.int8: torch.quint8, torch.qint8: torch.quint8, torch.uint8: torch.quint8, torch.quint8: torch.quint8, torch.quint4x2: torch.quint4x2,
            torch.quint2x4: torch.quint2x4, torch.float16: torch.float16, torch.float32: torch.float32}[dtype]


def quantize_feature(module: nn.Module, inputs: Tuple[torch.Tensor, ...]) -> Tuple[torch.Tensor, ...]:
    return tuple(i.half() if isinstance(i, torch.Tensor) and i.dtype in (torch.float32, torch.float64) else i for i in inputs)


def quantize_embeddings(module: nn.Module, dtype: torch.dtype, inplace: bool, additional_qconfig_spec_keys: Optional[List[Type[nn.Module]]] = None,
                        additional_mapping: Optional[Dict[Type[nn.Module], Type[nn.Module]]] = None, output_dtype: torch.dtype = torch.float,
                        per_table_weight_dtype: Optional[Dict[str, torch.dtype]] = None) -> nn.Module:
    """Swap every ``EmbeddingBagCollection`` / ``EmbeddingCollection`` under ``module`` for its quantized counterpart."""
    qconfig = QuantConfig(activation=tq.PlaceholderObserver.with_args(dtype=output_dtype), weight=tq.PlaceholderObserver.with_args(dtype=_qdtype(dtype)),
                          per_table_weight_dtype=per_table_weight_dtype)
    mapping: Dict[Type[nn.Module], Type[nn.Module]] = {EmbeddingBagCollection: QuantEmbeddingBagCollection, EmbeddingCollection: QuantEmbeddingCollection}
    if additional_mapping:
        mapping.update(additional_mapping)
    root = module if inplace else copy.deepcopy(module)

    def convert(parent: nn.Module) -> None:
        for name, child in list(parent.named_children()):
            if type(child) in mapping:
                child.qconfig = qconfig
                setattr(parent, name, mapping[type(child)].from_float(child))
            else:
                convert(child)

    if type(root) in mapping:
        root.qconfig = qconfig
        return mapping[type(root)].from_float(root)
    convert(root)
    return root


@dataclass
class QualNameMetadata:
    need_preproc: bool


@dataclass
class BatchingMetadata:
    """How the serving runtime batches one model input: ``type`` ("dense" / "sparse" / "unit"), the ``device`` it is
    staged on and the names of the inputs it must be pinned with."""

    type: str
    device: str
    pinned: List[str]


class PredictFactory(abc.ABC):
    """What a model owner implements to hand a model to the serving runtime."""

    @abc.abstractmethod
    def create_predict_module(self) -> nn.Module:
        """The module to serve (already quantized / sharded as desired)."""

    @abc.abstractmethod
    def batching_metadata(self) -> Dict[str, BatchingMetadata]:
        """Per model input: how to batch it."""

    def batching_metadata_json(self) -> str:
        import json

        return json.dumps({k: {"type": v.type, "device": v.device, "pinned": v.pinned} for k, v in self.batching_metadata().items()})

    @abc.abstractmethod
    def result_metadata(self) -> str:
        """Name of the result splitter ("dict_of_tensor", ...)."""

    @abc.abstractmethod
    def run_weights_independent_tranformations(self, predict_module: nn.Module) -> nn.Module:
        """Transformations that do not need the trained weights (fx passes, ...)."""

    @abc.abstractmethod
    def run_weights_dependent_transformations(self, predict_module: nn.Module) -> nn.Module:
        """Transformations that need the weights (quantization, sharding)."""

    def qualname_metadata(self) -> Dict[str, QualNameMetadata]:
        return {}

    def qualname_metadata_json(self) -> str:
        import json

        return json.dumps({k: {"need_preproc": v.need_preproc} for k, v in self.qualname_metadata().items()})

    def model_inputs_data(self) -> Dict[str, Any]:
        return {}


class PredictModule(nn.Module):
    """Serving wrapper: moves the batch to the model's device, runs it without autograd, returns a dict of tensors."""

    def __init__(self, module: nn.Module, device: Optional[str] = None) -> None:
        super().__init__()
        self._module = module
        self._device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self._module.eval()

    @property
    def predict_module(self) -> nn.Module:
        return self._module

    @abc.abstractmethod
    def predict_forward(self, batch: Dict[str, torch.Tensor]) -> Any:
        ...

    def forward(self, batch: Dict[str, torch.Tensor]) -> Any:
        with torch.inference_mode():
            return self.predict_forward(batch)

    def state_dict(self, destination: Optional[Dict[str, Any]] = None, prefix: str = "", keep_vars: bool = False) -> Dict[str, Any]:
        # the served module's keys carry no wrapper prefix, so checkpoints of the bare model load directly
        return self._module.state_dict(destination=destination, prefix=prefix, keep_vars=keep_vars)


def quantize_dense(predict_module: PredictModule, dtype: torch.dtype, additional_embedding_module_type: List[Type[nn.Module]] = []) -> nn.Module:
    """Cast every non-embedding submodule to ``dtype`` (fp16 / bf16) and the float inputs with it."""
    module = predict_module
    skip = tuple([QuantEmbeddingBagCollection, QuantEmbeddingCollection, ShardedQuantEmbeddingBagCollection, ShardedQuantEmbeddingCollection,
                  EmbeddingBagCollection, EmbeddingCollection] + list(additional_embedding_module_type))

    def cast(m: nn.Module) -> None:
        for name, child in m.named_children():
            if isinstance(child, skip):
                continue
            if not any(isinstance(g, skip) for g in child.modules()):
                child.to(dtype)
            else:
                cast(child)

    cast(module)
    return predict_module


def set_pruning_data(model: nn.Module, tables_to_rows_post_pruning: Dict[str, int], module_types: Optional[List[Type[nn.Module]]] = None) -> nn.Module:
    module_types = module_types or [EmbeddingBagCollection, EmbeddingCollection]
    for m in model.modules():
        if type(m) in module_types:
            setattr(m, MODULE_ATTR_EMB_CONFIG_NAME_TO_NUM_ROWS_POST_PRUNING_DICT, tables_to_rows_post_pruning)
    return model


def quantize_inference_model(model: nn.Module, quantization_mapping: Optional[Dict[str, Type[nn.Module]]] = None,
                             per_table_weight_dtype: Optional[Dict[str, torch.dtype]] = None, fp_weight_dtype: torch.dtype = DEFAULT_QUANTIZATION_DTYPE,
                             quantization_dtype: torch.dtype = DEFAULT_QUANTIZATION_DTYPE, output_dtype: torch.dtype = torch.float) -> nn.Module:
    """Quantize all embedding collections of ``model`` in place (state dicts expose payload + scale/bias separately)."""
    for m in model.modules():
        if isinstance(m, (EmbeddingBagCollection, EmbeddingCollection)):
            quant_prep_enable_quant_state_dict_split_scale_bias(m)
    quant_prep_enable_register_tbes(model, [EmbeddingBagCollection, EmbeddingCollection])
    return quantize_embeddings(model, dtype=quantization_dtype, inplace=True, output_dtype=output_dtype, per_table_weight_dtype=per_table_weight_dtype)


def shard_quant_model(model: nn.Module, world_size: int = 1, compute_device: str = "cuda", sharding_device: str = "meta", sharders: Optional[List[Any]] = None,
                      device_memory_size: Optional[int] = None, constraints: Optional[Dict[str, Any]] = None, ddr_cap: Optional[int] = None) -> Tuple[nn.Module, ShardingPlan]:
    """Place the quantized tables of ``model`` on ``world_size`` devices of this host and swap the quantized modules for their sharded
    form.  Default: table-wise, largest table first onto the lightest device.  A table whose entry in ``constraints`` (an object with
    ``sharding_types``, e.g. ``ParameterConstraints``) asks for ``row_wise`` or ``column_wise`` first is placed that way; with ``device_memory_size`` (bytes per device) a table that does not fit on the
    lightest device is split row-wise over all devices."""
    env = ShardingEnv.from_local(world_size=world_size, rank=0)
    device = torch.device(compute_device)
    plan: Dict[str, Dict[str, ParameterSharding]] = {}
    load = [0] * world_size
    targets = []
    for path, m in model.named_modules():
        if isinstance(m, (QuantEmbeddingBagCollection, QuantEmbeddingCollection)):
            targets.append((path, m))
    sized = []
    for path, m in targets:
        container = m.embedding_bags if isinstance(m, QuantEmbeddingBagCollection) else m.embeddings
        for name, holder in container.items():
            sized.append((holder.weight.numel(), path, name))
    dims = {}
    for path, m in targets:
        for cfg in (m.embedding_bag_configs() if isinstance(m, QuantEmbeddingBagCollection) else m.embedding_configs()):
            dims[(path, cfg.name)] = cfg.embedding_dim
    for nbytes, path, name in sorted(sized, reverse=True):
        wanted = getattr((constraints or {}).get(name), "sharding_types", None) or [ShardingType.TABLE_WISE.value]
        if device_memory_size is not None and wanted[0] == ShardingType.TABLE_WISE.value and min(load) + nbytes > device_memory_size:
            wanted = [ShardingType.ROW_WISE.value]  # does not fit on any single device next to what is already there: split its rows
        if wanted[0] == ShardingType.ROW_WISE.value and world_size > 1:
            # equal row blocks on every device
            for i in range(world_size):
                load[i] += nbytes // world_size
            plan.setdefault(path, {})[name] = ParameterSharding(sharding_type=ShardingType.ROW_WISE.value, compute_kernel="quant", ranks=list(range(world_size)))
            continue
        if wanted[0] == ShardingType.COLUMN_WISE.value and world_size > 1:
            # as many equal column ranges as divide the width in multiples of 16, on the lightest devices
            n = max((k for k in range(1, world_size + 1) if dims[(path, name)] % (16 * k) == 0), default=1)
            ranks = sorted(range(world_size), key=lambda i: load[i])[:n]
            for i in ranks:
                load[i] += nbytes // n
            plan.setdefault(path, {})[name] = ParameterSharding(sharding_type=ShardingType.COLUMN_WISE.value if n > 1 else ShardingType.TABLE_WISE.value,
                                                                compute_kernel="quant", ranks=ranks)
            continue
        r = min(range(world_size), key=lambda i: load[i])
        load[r] += nbytes
        plan.setdefault(path, {})[name] = ParameterSharding(sharding_type=ShardingType.TABLE_WISE.value, compute_kernel="quant", ranks=[r])
    for path, m in targets:
        cls = ShardedQuantEmbeddingBagCollection if isinstance(m, QuantEmbeddingBagCollection) else ShardedQuantEmbeddingCollection
        sharded = cls(m, plan[path], env, device=device)
        if path == "":
            model = sharded
        else:
            parent = model
            parts = path.split(".")
            for p in parts[:-1]:
                parent = getattr(parent, p)
            setattr(parent, parts[-1], sharded)
    return model, ShardingPlan(plan)


def get_table_to_weights_from_tbe(model: nn.Module) -> Dict[str, List[Tuple[torch.Tensor, Optional[torch.Tensor]]]]:
    """``{table: [(packed weight, None)]}`` of every quantized table found under ``model`` (for weight hot-swap)."""
    out: Dict[str, List[Tuple[torch.Tensor, Optional[torch.Tensor]]]] = {}
    for m in model.modules():
        if isinstance(m, (QuantEmbeddingBagCollection, QuantEmbeddingCollection)):
            container = m.embedding_bags if isinstance(m, QuantEmbeddingBagCollection) else m.embeddings
            for name, holder in container.items():
                out.setdefault(name, []).append((holder.weight, None))
    return out


def assign_weights_to_tbe(model: nn.Module, table_to_weight: Dict[str, List[Tuple[torch.Tensor, Optional[torch.Tensor]]]]) -> None:
    """Copy packed tables into the model's lookup buffers in place (hot-swap of a new snapshot)."""
    current = get_table_to_weights_from_tbe(model)
    for name, dsts in current.items():
        srcs = table_to_weight.get(name)
        if srcs is None:
            continue
        for (dst, _), (src, _) in zip(dsts, srcs):
            dst.copy_(src.to(dst.device))
