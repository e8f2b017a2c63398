"""Utilities of the sharding runtime (cf. ``torchrec/distributed/utils.py``)."""
from __future__ import annotations

import copy
import logging
import pdb
import sys
from collections import OrderedDict
from contextlib import nullcontext
from typing import Any, Dict, List, Optional, Set, Type, TypeVar, Union

import torch
from torch import nn
from torch.autograd.profiler import record_function

from torchrec_b200 import optim as trec_optim
from torchrec_b200.distributed.embedding_types import EmbeddingComputeKernel
from torchrec_b200.distributed.types import DataType, EmbeddingEvent, ParameterSharding, ShardedModule, ShardingType
from torchrec_b200.ops.tbe import EmbOptimType
from torchrec_b200.types import CopyMixIn

logger: logging.Logger = logging.getLogger(__name__)
_T = TypeVar("_T")


def none_throws(optional: Optional[_T], message: str = "Unexpected `None`") -> _T:
    if optional is None:
        raise AssertionError(message)
    return optional


def append_prefix(prefix: str, name: str) -> str:
    """``"a." + "b" -> "a.b"``; empty parts are skipped."""
    if prefix != "" and name != "":
        return prefix + "." + name
    return prefix + name


def filter_state_dict(state_dict: "OrderedDict[str, torch.Tensor]", name: str) -> "OrderedDict[str, torch.Tensor]":
    """Entries whose key starts with ``name.``, with that prefix removed."""
    filtered = OrderedDict()
    for key, value in state_dict.items():
        if key.startswith(name + "."):
            filtered[key[len(name) + 1:]] = value
    return filtered


def add_prefix_to_state_dict(state_dict: Dict[str, Any], prefix: str) -> None:
    """In place: every key (and every non-empty key of the ``_metadata`` entry) gets ``prefix`` in front."""
    renamed = [(key, prefix + key) for key in sorted(state_dict)]
    for old, new in renamed:
        state_dict[new] = state_dict.pop(old)
    meta = state_dict.get("_metadata")
    if meta is not None:
        for old in [k for k in meta if k]:
            meta[prefix + old] = meta.pop(old)


def _get_unsharded_module_names_helper(model: nn.Module, path: str, unsharded_module_names: Set[str]) -> bool:
    """Returns whether ``model`` contains a sharded module.  When it does, its children that do not are reported (their own
    descendants need no separate entry); when it does not, the caller reports ``model`` itself."""
    holds_shards = {
        name: isinstance(child, ShardedModule) or _get_unsharded_module_names_helper(child, f"{path}{name}.", unsharded_module_names)
        for name, child in model.named_children()
    }
    if not any(holds_shards.values()):
        return False
    unsharded_module_names.update(path + name for name, has in holds_shards.items() if not has)
    return True


def get_unsharded_module_names(model: nn.Module) -> List[str]:
    """Minimal set of module paths that contain no sharded submodule."""
    unsharded: Set[str] = set()
    _get_unsharded_module_names_helper(model, "", unsharded)
    return list(unsharded)


class sharded_model_copy:
    """Context manager: ``copy.deepcopy`` of a sharded model keeps sharded tensors on ``device``
    (e.g. ``with sharded_model_copy("cpu"): m_cpu = copy.deepcopy(m)``).  It works by swapping the ``__deepcopy__`` of tensors
    and parameters for the duration of the block."""

    def __init__(self, device: Optional[Union[str, int, torch.device]]) -> None:
        self.device = device
        self._saved: Optional[tuple] = None

    def _clone(self, tensor: torch.Tensor, memo) -> torch.Tensor:
        detached = tensor.detach()
        return detached.clone() if tensor.device == self.device else detached.to(self.device)

    def __enter__(self) -> None:
        self._saved = (torch.Tensor.__deepcopy__, torch.nn.Parameter.__deepcopy__)
        clone = self._clone
        torch.Tensor.__deepcopy__ = lambda t, memo: clone(t, memo)
        torch.nn.Parameter.__deepcopy__ = lambda p, memo: torch.nn.Parameter(clone(p, memo), requires_grad=p.requires_grad)

    def __exit__(self, exc_type, exc_val, exc_tb) -> None:
        torch.Tensor.__deepcopy__, torch.nn.Parameter.__deepcopy__ = self._saved


def copy_to_device(module: nn.Module, current_device: torch.device, to_device: torch.device) -> nn.Module:
    """Deep copy of ``module`` in which everything that lives on ``current_device`` moves to ``to_device``; tensors on other
    devices (sharded tables) are shared with the original through ``sharded_model_copy``."""
    with sharded_model_copy(device=None):
        twin = copy.deepcopy(module)
    if isinstance(twin, CopyMixIn):
        return twin.copy(to_device)

    def moved(t: torch.Tensor) -> torch.Tensor:
        return t.to(to_device) if t.device == current_device else t

    for name, p in list(twin.named_parameters(recurse=False)):
        twin.register_parameter(name, torch.nn.Parameter(moved(p.data), requires_grad=p.requires_grad))
    for name, buf in list(twin.named_buffers(recurse=False)):
        twin.register_buffer(name, moved(buf))
    for name, child in list(twin.named_children()):
        if isinstance(child, CopyMixIn) or any(p.device == current_device for p in child.parameters()):
            setattr(twin, name, copy_to_device(child, current_device, to_device))
    return twin


def optimizer_type_to_emb_opt_type(optimizer_class: Type[torch.optim.Optimizer]) -> Optional[EmbOptimType]:
    """Which fused kernel update an optimizer class selects."""
    from torchrec_b200.optim import optimizers as marker
    from torchrec_b200.optim.rowwise_adagrad import RowWiseAdagrad

    lookup = {
        torch.optim.SGD: EmbOptimType.EXACT_SGD,
        torch.optim.Adagrad: EmbOptimType.EXACT_ADAGRAD,
        torch.optim.Adam: EmbOptimType.ADAM,
        marker.SGD: EmbOptimType.EXACT_SGD,
        marker.LarsSGD: EmbOptimType.LARS_SGD,
        marker.LAMB: EmbOptimType.LAMB,
        marker.PartialRowWiseLAMB: EmbOptimType.PARTIAL_ROWWISE_LAMB,
        marker.Adam: EmbOptimType.ADAM,
        marker.PartialRowWiseAdam: EmbOptimType.PARTIAL_ROWWISE_ADAM,
        marker.Adagrad: EmbOptimType.EXACT_ADAGRAD,
        RowWiseAdagrad: EmbOptimType.EXACT_ROWWISE_ADAGRAD,
    }
    if optimizer_class not in lookup:
        raise ValueError(f"Cannot cast {optimizer_class} to an EmbOptimType")
    return lookup[optimizer_class]


def merge_fused_params(fused_params: Optional[Dict[str, Any]] = None, param_fused_params: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
    """Sharder-level fused params overridden by the per-parameter optimizer kwargs (``lr`` -> ``learning_rate``)."""
    merged = copy.deepcopy(fused_params or {})
    overrides = param_fused_params if param_fused_params is not None else {}
    if "lr" in overrides:
        overrides["learning_rate"] = overrides.pop("lr")  # the kernels know the learning rate under this name
    merged.update(overrides)
    return merged


def add_params_from_parameter_sharding(fused_params: Optional[Dict[str, Any]], parameter_sharding: ParameterSharding) -> Dict[str, Any]:
    if fused_params is None:
        fused_params = {}
    if parameter_sharding.cache_params is not None:
        cp = parameter_sharding.cache_params
        for name in ("algorithm", "load_factor", "reserved_memory", "precision", "prefetch_pipeline", "multipass_prefetch_config"):
            v = getattr(cp, name)
            if v is not None:
                fused_params[{"algorithm": "cache_algorithm", "load_factor": "cache_load_factor", "reserved_memory": "cache_reserved_memory", "precision": "cache_precision"}.get(name, name)] = v
    for name in ("enforce_hbm", "stochastic_rounding", "bounds_check_mode", "output_dtype"):
        v = getattr(parameter_sharding, name)
        if v is not None:
            fused_params[name] = v
    if parameter_sharding.compute_kernel in {EmbeddingComputeKernel.KEY_VALUE.value, EmbeddingComputeKernel.SSD_VIRTUAL_TABLE.value, EmbeddingComputeKernel.DRAM_VIRTUAL_TABLE.value}:
        kv = parameter_sharding.key_value_params
        if kv is not None:
            for k, v in kv.__dict__.items():
                if v is not None:
                    fused_params[k] = v
    return fused_params


def convert_to_fbgemm_types(fused_params: Dict[str, Any]) -> Dict[str, Any]:
    """Kept for API parity: kernel-side enums are native to this package, nothing to convert."""
    return fused_params


def init_parameters(module: nn.Module, device: torch.device) -> None:
    """Materialise ``meta`` parameters on ``device`` and run ``reset_parameters`` where defined."""
    with torch.no_grad():
        has_meta_param = any(isinstance(p, torch.Tensor) and p.device.type == "meta" for p in module._parameters.values())
        for key, buf in list(module._buffers.items()):
            if isinstance(buf, torch.Tensor) and buf.device.type == "meta":
                module._buffers[key] = torch.zeros_like(buf, device=device)
        if has_meta_param:
            for key, param in list(module._parameters.items()):
                if isinstance(param, torch.Tensor) and param.device.type == "meta":
                    module._parameters[key] = nn.Parameter(torch.empty_like(param, device=device), requires_grad=param.requires_grad)

        def maybe_reset(m: nn.Module) -> None:
            if has_meta_param and hasattr(m, "reset_parameters"):
                m.reset_parameters()

        maybe_reset(module)


def maybe_annotate_embedding_event(event: EmbeddingEvent, module_fqn: Optional[str], sharding_type: Optional[str]):
    """Profiler range ``## <event>: [<module>, <sharding>] ##`` when both names are known."""
    if module_fqn and sharding_type:
        return record_function(f"## {event.value}: [{module_fqn}, {sharding_type}] ##")
    return nullcontext()


class ForkedPdb(pdb.Pdb):
    """pdb usable inside a spawned rank (re-opens stdin)."""

    def interaction(self, *args, **kwargs) -> None:
        _stdin = sys.stdin
        try:
            sys.stdin = open("/dev/stdin")
            pdb.Pdb.interaction(self, *args, **kwargs)
        finally:
            sys.stdin = _stdin


def modify_input_for_feature_processor(features, feature_processors, is_collection: bool) -> None:
    """Give unweighted features unit weights so that position-weighted processors can scale them."""
    with torch.no_grad():
        if features.weights_or_none() is None:
            cat_weights = torch.ones(features.values().numel(), dtype=torch.float32, device=features.device())
            features._weights = cat_weights


# ---- small helpers of the reference's ``distributed/utils.py`` ---------------------------------------------------------------
_T = TypeVar("_T")


def get_device_type() -> str:
    return "cuda" if torch.cuda.is_available() else "cpu"


def get_class_name(obj: object) -> str:
    return "None" if obj is None else type(obj).__name__


def assert_instance(obj: object, t: Type[_T]) -> _T:
    assert isinstance(obj, t), f"Got {get_class_name(obj)}"
    return obj


class CopyableMixin(nn.Module):
    """``module.copy(device)``: a copy of a host-resident module on ``device`` (sharded submodules copy themselves through their own
    ``copy`` hook, see ``copy_to_device``)."""

    def copy(self, device: torch.device) -> nn.Module:
        return copy_to_device(self, current_device=torch.device("cpu"), to_device=device)


def create_global_tensor_shape_stride_from_metadata(parameter_sharding: ParameterSharding, devices_per_node: Optional[int] = None):
    """``(shape, stride)`` of the whole table that the shards of ``parameter_sharding`` tile."""
    shards = parameter_sharding.sharding_spec.shards
    kind = parameter_sharding.sharding_type
    rows, cols = shards[0].shard_sizes
    if kind == ShardingType.COLUMN_WISE.value or kind == ShardingType.TABLE_COLUMN_WISE.value:
        cols = sum(s.shard_sizes[1] for s in shards)
    elif kind in (ShardingType.ROW_WISE.value, ShardingType.TABLE_ROW_WISE.value):
        rows = sum(s.shard_sizes[0] for s in shards)
    elif kind == ShardingType.GRID_SHARD.value:
        assert devices_per_node is not None, "grid shards need the node size to tell row shards from column shards"
        rows, cols = rows * devices_per_node, cols * (len(shards) // devices_per_node)
    elif kind != ShardingType.TABLE_WISE.value:
        return torch.Size([0, 0]), (0, 1)
    return torch.Size([rows, cols]), (cols, 1)


def get_bucket_metadata_from_shard_metadata(shards, num_buckets: int):
    """Bucket layout of a row-wise table cut into ``num_buckets`` equal buckets, every shard holding whole buckets."""
    from torchrec_b200.distributed.types import ShardingBucketMetadata

    assert len(shards) > 0, "Shards cannot be empty"
    table_rows = shards[-1].shard_offsets[0] + shards[-1].shard_sizes[0]
    assert table_rows % num_buckets == 0, f"Table size '{table_rows}' must be divisible by num_buckets '{num_buckets}'"
    bucket = table_rows // num_buckets
    meta = ShardingBucketMetadata(num_buckets_per_shard=[], bucket_offsets_per_shard=[], bucket_size=bucket)
    first = 0
    for shard in shards:
        assert len(shard.shard_offsets) == 1 or shard.shard_offsets[1] == 0, "only row-wise shards can be bucketized"
        assert shard.shard_sizes[0] % bucket == 0, f"Shard size[0] '{shard.shard_sizes[0]}' is not divisible by bucket size '{bucket}'"
        meta.num_buckets_per_shard.append(shard.shard_sizes[0] // bucket)
        meta.bucket_offsets_per_shard.append(first)
        first += shard.shard_sizes[0] // bucket
    return meta


def weights_bytes_in_emb_kernel(emb: nn.Module) -> int:
    """Bytes of table storage held by one embedding kernel."""
    w = getattr(emb, "weights", None)
    return int(w.numel() * w.element_size()) if isinstance(w, torch.Tensor) else sum(int(t.numel() * t.element_size()) for t in emb.split_embedding_weights())
