"""``DistributedModelParallel``: the entry point that shards a model.

It plans (collectively, unless a plan is given), swaps every shardable submodule for its sharded
counterpart, materialises the remaining ``meta`` parameters on the device, wraps the unsharded rest
in ``DistributedDataParallel`` and exposes a ``state_dict`` whose keys equal the unsharded model's.
``DMPCollection`` adds 2D parallelism: model-parallel inside a sharding group, replicated across
groups with periodic weight/optimizer-state averaging.

Counterpart of ``torchrec/distributed/model_parallel.py`` (``DistributedModelParallel`` ``:196``,
``DefaultDataParallelWrapper`` ``:83``, ``DMPCollection`` ``:785``).
"""
from __future__ import annotations

import abc
import copy
import logging as logger
from collections import OrderedDict
from typing import Any, Dict, Iterator, List, Optional, Set, Tuple, Type, Union, cast

import torch
import torch.distributed as dist
from torch import nn
from torch.distributed.algorithms.ddp_comm_hooks import default_hooks as ddp_default_hooks
from torch.nn.modules.module import _IncompatibleKeys
from torch.nn.parallel import DistributedDataParallel

from torchrec_b200.distributed.comm import get_local_size
from torchrec_b200.distributed.sharding_plan import get_default_sharders
from torchrec_b200.distributed.types import (
    DMPCollectionConfig,
    DMPCollectionContext,
    EmbeddingModuleShardingPlan,
    ModuleSharder,
    ParameterSharding,
    ShardedModule,
    ShardingEnv,
    ShardingEnv2D,
    ShardingPlan,
)
from torchrec_b200.distributed.utils import (
    add_prefix_to_state_dict,
    append_prefix,
    copy_to_device,
    filter_state_dict,
    init_parameters,
    sharded_model_copy,
)
from torchrec_b200.optim.fused import FusedOptimizerModule
from torchrec_b200.optim.keyed import CombinedOptimizer, KeyedOptimizer

_DDP_STATE_DICT_PREFIX = "module."
_FSDP_WRAPPED_MODULE = "_fsdp_wrapped_module"


class DataParallelWrapper(abc.ABC):
    """Strategy that wraps the non-sharded part of a model for data parallelism."""

    @abc.abstractmethod
    def wrap(self, dmp: "DistributedModelParallel", env: ShardingEnv, device: torch.device) -> None:
        ...


_COMPRESSION_HOOKS = {"fp16": ddp_default_hooks.fp16_compress_hook, "bf16": ddp_default_hooks.bf16_compress_hook}


class DefaultDataParallelWrapper(DataParallelWrapper):
    """DDP over every parameter that is not owned by a sharded module.

    25 MB buckets, static graph, gradients as bucket views; optional fp16 / bf16 gradient compression.
    (``PeerDataParallelWrapper`` in ``peer_data_parallel.py`` is the single-node alternative that needs no DDP.)
    """

    def __init__(self, bucket_cap_mb: int = 25, static_graph: bool = True, find_unused_parameters: bool = False,
                 allreduce_comm_precision: Optional[str] = None, params_to_ignore: Optional[List[str]] = None,
                 ddp_kwargs: Optional[Dict[str, Any]] = None) -> None:
        self._ddp_options: Dict[str, Any] = dict(bucket_cap_mb=bucket_cap_mb, static_graph=static_graph, find_unused_parameters=find_unused_parameters,
                                                 gradient_as_bucket_view=True, broadcast_buffers=False)
        self._ddp_options.update(ddp_kwargs or {})
        self._allreduce_comm_precision = allreduce_comm_precision
        self._additional_params_to_ignore: Set[str] = set(params_to_ignore or [])

    def _ddp_wrap(self, dmp: "DistributedModelParallel", env: ShardingEnv, device: torch.device, ddp_ignore_param_names: Set[str]) -> None:
        if env.process_group is None:
            raise RuntimeError("Can only init DDP for ProcessGroup-based ShardingEnv")
        trainable = {name for name, p in dmp.named_parameters() if p.requires_grad}
        if trainable <= ddp_ignore_param_names:
            return  # nothing left to average (e.g. a model that is all embedding tables)
        inner = dmp._dmp_wrapped_module
        DistributedDataParallel._set_params_and_buffers_to_ignore_for_model(module=inner, params_and_buffers_to_ignore=ddp_ignore_param_names)
        ddp = DistributedDataParallel(module=inner.to(device), device_ids=[device] if device.type != "cpu" else None,
                                      process_group=env.process_group, **self._ddp_options)
        hook = _COMPRESSION_HOOKS.get(self._allreduce_comm_precision or "")
        if hook is not None:
            ddp.register_comm_hook(None, hook)
        dmp._dmp_wrapped_module = cast(nn.Module, ddp)

    def wrap(self, dmp: "DistributedModelParallel", env: ShardingEnv, device: torch.device) -> None:
        if isinstance(dmp._dmp_wrapped_module, DistributedDataParallel):
            return
        owned_by_shards = set(DistributedModelParallel._sharded_parameter_names(dmp._dmp_wrapped_module))
        self._ddp_wrap(dmp, env, device, owned_by_shards | self._additional_params_to_ignore)


def _strip(module: nn.Module, ddp_too: bool) -> nn.Module:
    while True:
        if isinstance(module, DistributedModelParallel):
            module = module._dmp_wrapped_module
        elif ddp_too and isinstance(module, DistributedDataParallel):
            module = module.module
        else:
            return module


def get_unwrapped_module(module: nn.Module) -> nn.Module:
    """Strip ``DistributedModelParallel`` / DDP wrappers."""
    return _strip(module, ddp_too=True)


def get_module(module: nn.Module) -> nn.Module:
    """Strip ``DistributedModelParallel`` wrappers only (data-parallel wrappers stay)."""
    return _strip(module, ddp_too=False)


def _join(prefix: str, name: str) -> str:
    return f"{prefix}.{name}" if prefix else name


def _leaves(module: nn.Module, prefix: str = "") -> Iterator[Tuple[str, nn.Module, bool]]:
    """Depth-first walk that stops at sharded modules: yields ``(path, module, is_sharded)`` for every module visited,
    with data-parallel wrappers looked through (so paths are those of the unsharded model)."""
    module = get_unwrapped_module(module)
    sharded = isinstance(module, ShardedModule)
    yield prefix, module, sharded
    if not sharded:
        for name, child in module.named_children():
            yield from _leaves(child, append_prefix(prefix, name))


def _unique(pairs: Iterator[Tuple[str, Any]], remove_duplicate: bool) -> Iterator[Tuple[str, Any]]:
    seen = set()
    for name, t in pairs:
        if t in seen:
            continue
        if remove_duplicate:
            seen.add(t)
        yield name, t


class DistributedModelParallel(nn.Module, FusedOptimizerModule):
    """Shard ``module``'s embedding submodules over ``env`` and data-parallelise the rest.

    Args:
        module: model to wrap; embedding modules may live on the ``meta`` device.
        env: sharding environment (default: the world process group).
        device: compute device of this rank.
        plan: sharding plan; by default ``EmbeddingShardingPlanner.collective_plan`` is used.
        sharders: available sharders (default: ``get_default_sharders()``).
        init_data_parallel: wrap the dense part in DDP now (else call ``init_data_parallel()`` later).
        init_parameters: materialise and initialise parameters that are still on ``meta``.
        data_parallel_wrapper: custom wrapper for the dense part.
    """

    SHARE_SHARDED: bool = False
    SHARED_SHARDED_MODULE: Dict[str, ShardedModule] = {}

    def __init__(
        self,
        module: nn.Module,
        env: Optional[ShardingEnv] = None,
        device: Optional[torch.device] = None,
        plan: Optional[ShardingPlan] = None,
        sharders: Optional[List[ModuleSharder[torch.nn.Module]]] = None,
        init_data_parallel: bool = True,
        init_parameters: bool = True,
        data_parallel_wrapper: Optional[DataParallelWrapper] = None,
        model_tracker_config: Optional[Any] = None,
    ) -> None:
        super().__init__()
        self.init_parameters = init_parameters
        self._ddp_wrapped: bool = False
        self._env: ShardingEnv = env if env is not None else self._world_env()
        self.device: torch.device = device if device is not None else torch.device("cpu")
        sharders = sharders if sharders is not None else get_default_sharders()
        self._sharder_map: Dict[Type[nn.Module], ModuleSharder[nn.Module]] = {s.module_type: s for s in sharders}
        self._data_parallel_wrapper: DataParallelWrapper = data_parallel_wrapper or DefaultDataParallelWrapper()
        self._plan: ShardingPlan = plan if plan is not None else self._make_plan(module, sharders)
        self._dmp_wrapped_module: nn.Module = self._init_dmp(module)
        self._optim: CombinedOptimizer = self._init_optim(self._dmp_wrapped_module)
        if init_parameters:
            self._init_parameters(self.module)
        if init_data_parallel:
            self.init_data_parallel()
        self.model_delta_tracker = None if model_tracker_config is None else self._init_delta_tracker(model_tracker_config, self._dmp_wrapped_module)

    @staticmethod
    def _world_env() -> ShardingEnv:
        world = dist.GroupMember.WORLD
        assert world is not None, "Process group is not initialized"
        return ShardingEnv.from_process_group(world)

    def _make_plan(self, module: nn.Module, sharders: List[ModuleSharder[nn.Module]]) -> ShardingPlan:
        from torchrec_b200.distributed.planner import EmbeddingShardingPlanner, Topology

        topology = Topology(local_world_size=get_local_size(self._env.world_size), world_size=self._env.world_size, compute_device=self.device.type)
        planner = EmbeddingShardingPlanner(topology=topology)
        group = self._env.process_group
        return planner.plan(module, sharders) if group is None else planner.collective_plan(module, sharders, group)

    @property
    def module(self) -> nn.Module:
        """The wrapped module with DDP wrappers removed."""
        return get_unwrapped_module(self)

    @module.setter
    def module(self, value: nn.Module) -> None:
        if isinstance(self.module, DistributedDataParallel):
            raise RuntimeError("module can't be set after calling init_data_parallel(...)")
        self._dmp_wrapped_module = value

    def forward(self, *args, **kwargs) -> Any:
        return self._dmp_wrapped_module(*args, **kwargs)

    def init_data_parallel(self) -> None:
        """Wrap the dense part (deferred form of ``init_data_parallel=True``); idempotent."""
        if self._ddp_wrapped:
            return
        self._data_parallel_wrapper.wrap(self, self._env, self.device)
        self._ddp_wrapped = True

    def copy(self, device: torch.device) -> "DistributedModelParallel":
        """Copy of the wrapper whose dense part lives on ``device``; sharded modules are shared."""
        assert isinstance(device, torch.device)
        with sharded_model_copy(device=None):
            twin = copy.deepcopy(self)
        twin._dmp_wrapped_module = copy_to_device(self._dmp_wrapped_module, self.device, device)
        return twin

    # ---- construction steps ---------------------------------------------------------------------------------------------------
    def _init_dmp(self, module: nn.Module) -> nn.Module:
        return self._shard_modules_impl(module)

    def _init_delta_tracker(self, config, module):
        from torchrec_b200.distributed.model_tracker.model_delta_tracker import ModelDeltaTracker

        return ModelDeltaTracker(model=module, consumers=getattr(config, "consumers", None), delete_on_read=getattr(config, "delete_on_read", True),
                                 auto_compact=getattr(config, "auto_compact", False), mode=getattr(config, "tracking_mode", None),
                                 fqns_to_skip=getattr(config, "fqns_to_skip", ()))

    def get_model_tracker(self):
        assert self.model_delta_tracker is not None, "Model tracker is not initialized. Add ModelTrackerConfig at DistributedModelParallel init."
        return self.model_delta_tracker

    def get_delta(self, consumer: Optional[str] = None):
        assert self.model_delta_tracker is not None, "Model tracker is not initialized."
        return self.model_delta_tracker.get_delta(consumer)

    def _init_optim(self, module: nn.Module) -> CombinedOptimizer:
        return CombinedOptimizer(self._fused_optim_impl(module, []))

    def _fused_optim_impl(self, module: nn.Module, fused_optims: List[Tuple[str, KeyedOptimizer]], path: str = "") -> List[Tuple[str, KeyedOptimizer]]:
        """Fused optimizers of the tree, keyed by the path of the module that owns them (a module that owns one is a leaf)."""
        stack = [(path, module)]
        found: List[Tuple[str, KeyedOptimizer]] = []
        while stack:
            where, m = stack.pop()
            if isinstance(m, FusedOptimizerModule):
                found.append((where, m.fused_optimizer))
            else:
                stack.extend((_join(where, n), c) for n, c in reversed(list(m.named_children())))
        fused_optims.extend(found)
        return fused_optims

    def _shard_modules_impl(self, module: nn.Module, path: str = "") -> nn.Module:
        """Replace every module the plan names by its sharded form, top-down (a replaced module is not descended into)."""
        if isinstance(module, ShardedModule):
            return module
        plan_here = self._plan.get_plan_for_module(path)
        if plan_here:
            sharded = self._sharder_map[type(module)].shard(module, plan_here, self._env, self.device, path)
            torch._C._log_api_usage_once(f"torchrec.distributed.{type(sharded).__name__}")
            return sharded
        for name, child in list(module.named_children()):
            replacement = self._shard_modules_impl(child, _join(path, name))
            if replacement is not child:
                setattr(module, name, replacement)
        return module

    def _init_parameters(self, module: nn.Module) -> None:
        with torch.no_grad():
            for _, m, sharded in _leaves(module):
                if not sharded:
                    init_parameters(m, self.device)

    # ---- named members with DDP prefixes removed and sharded modules reported under unsharded names ----
    def sparse_grad_parameter_names(self, destination: Optional[List[str]] = None, prefix: str = "") -> List[str]:
        return self._sparse_grad_parameter_names(self.module, [] if destination is None else destination, prefix)

    def _sparse_grad_parameter_names(self, module: nn.Module, destination: List[str], prefix: str = "") -> List[str]:
        for where, m, sharded in _leaves(module, prefix):
            if not sharded and isinstance(m, (nn.Embedding, nn.EmbeddingBag)) and m.sparse:
                destination.append(append_prefix(where, "weight"))
        return destination

    def state_dict(self, destination: Optional[Dict[str, Any]] = None, prefix: str = "", keep_vars: bool = False) -> Dict[str, Any]:
        sd = get_module(self).state_dict(destination=destination, prefix=prefix, keep_vars=keep_vars)
        # keys of the unsharded model: no "module." of a data-parallel wrapper
        torch.nn.modules.utils.consume_prefix_in_state_dict_if_present(sd, prefix + _DDP_STATE_DICT_PREFIX)
        add_prefix_to_state_dict(sd, prefix)
        return sd

    def load_state_dict(self, state_dict: "OrderedDict[str, torch.Tensor]", prefix: str = "", strict: bool = True) -> _IncompatibleKeys:
        return self._load_state_dict(self, state_dict, prefix, strict)

    def _load_state_dict(self, module: nn.Module, state_dict: "OrderedDict[str, torch.Tensor]", prefix: str = "", strict: bool = True) -> _IncompatibleKeys:
        module = get_module(module)
        if isinstance(module, DistributedDataParallel):
            torch.nn.modules.utils.consume_prefix_in_state_dict_if_present(state_dict, prefix)
            add_prefix_to_state_dict(state_dict, prefix + _DDP_STATE_DICT_PREFIX)
        if getattr(module, "_FORCE_STATE_DICT_LOAD", False):
            return module.load_state_dict(state_dict, strict=strict)
        missing: List[str] = []
        unexpected: List[str] = []
        module._load_from_state_dict(state_dict, prefix, {}, strict, missing, unexpected, [])
        for name, child in module.named_children():
            sub = self._load_state_dict(child, filter_state_dict(state_dict, prefix + name), "", strict)
            missing += sub.missing_keys
            unexpected += sub.unexpected_keys
        return _IncompatibleKeys(missing_keys=missing, unexpected_keys=unexpected)

    def _named_parameters(self, module: nn.Module, prefix: str = "", recurse: bool = True, strip_ddp: bool = True) -> Iterator[Tuple[str, torch.nn.Parameter]]:
        if not strip_ddp and isinstance(module, DistributedDataParallel):
            yield from module.named_parameters(prefix, recurse=False)
            for name, child in module.named_children():
                yield from self._named_parameters(child, append_prefix(prefix, name), recurse, strip_ddp)
            return
        for where, m, sharded in _leaves(module, prefix):
            yield from m.named_parameters(where, recurse if sharded else False)

    def named_parameters(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True) -> Iterator[Tuple[str, torch.nn.Parameter]]:
        yield from _unique(self._named_parameters(self.module, prefix, recurse), remove_duplicate)

    def bare_named_parameters(self, prefix: str = "", recurse: bool = True) -> Iterator[Tuple[str, torch.nn.Parameter]]:
        yield from _unique(self._named_parameters(self.module, prefix, recurse), True)

    @staticmethod
    def _sharded_parameter_names(module: nn.Module, prefix: str = "") -> Iterator[str]:
        for where, m, sharded in _leaves(module, prefix):
            if sharded:
                yield from m.sharded_parameter_names(where)

    def _named_buffers(self, module: nn.Module, prefix: str = "", recurse: bool = True) -> Iterator[Tuple[str, torch.Tensor]]:
        for where, m, sharded in _leaves(module, prefix):
            yield from m.named_buffers(where, recurse if sharded else False)

    def named_buffers(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True) -> Iterator[Tuple[str, torch.Tensor]]:
        yield from _unique(self._named_buffers(self.module, prefix, recurse), remove_duplicate)

    @property
    def fused_optimizer(self) -> KeyedOptimizer:
        return self._optim

    @property
    def plan(self) -> ShardingPlan:
        return self._plan

    @staticmethod
    def _reset_parameters(module: nn.Module) -> None:
        for m in module.modules():
            reset = getattr(m, "reset_parameters", None)
            if reset is not None:
                reset()

    def reshard(self, sharded_module_fqn: str, changed_shard_to_params: Dict[str, ParameterSharding]) -> None:
        """Move the shards of ``sharded_module_fqn`` to a new placement at run time (dynamic resharding)."""
        from torchrec_b200.distributed.sharding.dynamic_sharding import reshard_module

        target = self.module.get_submodule(sharded_module_fqn)
        assert isinstance(target, ShardedModule)
        reshard_module(self, sharded_module_fqn, target, changed_shard_to_params)
        self._optim = self._init_optim(self._dmp_wrapped_module)
        self._plan.plan[sharded_module_fqn] = target.module_sharding_plan


def _rank_groups(world_size: int, group_size: int, contiguous: bool) -> Tuple[List[List[int]], List[List[int]]]:
    """(sharding groups, replica groups).  ``contiguous``: a sharding group is a run of consecutive ranks (one host) and its
    replicas are the ranks with the same position in other runs; otherwise sharding groups are strided over the world."""
    n_groups = world_size // group_size
    if contiguous:
        shard = [list(range(g * group_size, (g + 1) * group_size)) for g in range(n_groups)]
        replica = [list(range(i, world_size, group_size)) for i in range(group_size)]
    else:
        shard = [list(range(g, world_size, n_groups)) for g in range(n_groups)]
        replica = [list(range(i * n_groups, (i + 1) * n_groups)) for i in range(group_size)]
    return shard, replica


class DMPCollection(DistributedModelParallel):
    """2D parallelism: the world is split into sharding groups of ``sharding_group_size`` ranks; the
    model is sharded inside a group and the groups are replicas.  ``sync()`` averages embedding weights
    and fused optimizer state across replicas."""

    def __init__(
        self,
        module: nn.Module,
        device: torch.device,
        plan: ShardingPlan,
        world_size: int,
        sharding_group_size: int,
        global_pg: dist.ProcessGroup,
        node_group_size: Optional[int] = None,
        sharders: Optional[List[ModuleSharder[torch.nn.Module]]] = None,
        init_data_parallel: bool = True,
        init_parameters: bool = True,
        data_parallel_wrapper: Optional[DataParallelWrapper] = None,
        use_inter_host_allreduce: bool = False,
        custom_all_reduce: Optional[Any] = None,
        submodule_configs: Optional[List[DMPCollectionConfig]] = None,
    ) -> None:
        assert device.type in ("cuda", "cpu"), "DMPCollection needs a cuda or cpu device"
        assert sharding_group_size > 0 and world_size % sharding_group_size == 0, "sharding_group_size must divide the world size"
        self._global_pg, self._global_rank = global_pg, dist.get_rank(global_pg)
        self._device = device
        self._custom_all_reduce = custom_all_reduce
        self._use_inter_host_allreduce = use_inter_host_allreduce
        self._sharding_pg, self._replica_pg = self._create_process_groups(global_pg, world_size, sharding_group_size, use_inter_host_allreduce)
        self._remap_sharding_plan(plan, self._global_rank, world_size // sharding_group_size, use_inter_host_allreduce, sharding_group_size)
        env = ShardingEnv2D(self._sharding_pg, global_pg, None, node_group_size, use_inter_host_allreduce)
        super().__init__(module, env, device, plan, sharders, init_data_parallel, init_parameters, data_parallel_wrapper)
        self._modules_to_sync: List[nn.Module] = self._group_sharded_modules()

    @staticmethod
    def _create_process_groups(global_pg, world_size: int, sharding_group_size: int, inter_host: bool):
        """``sharding_pg``: ranks that shard together; ``replica_pg``: ranks holding the same shard.  Every rank creates
        every group (group creation is collective) and keeps the two it belongs to."""
        me, backend = dist.get_rank(global_pg), dist.get_backend(global_pg)
        mine: List[Optional[dist.ProcessGroup]] = []
        for family in _rank_groups(world_size, sharding_group_size, inter_host):
            kept = None
            for ranks in family:
                group = dist.new_group(ranks=ranks, backend=backend)
                kept = group if me in ranks else kept
            mine.append(kept)
        return mine[0], mine[1]

    @staticmethod
    def _remap_sharding_plan(plan: ShardingPlan, rank: int, step: int, inter_host: bool, sharding_group_size: int) -> None:
        """Plans are written for ranks ``0..group_size-1``; map them to the global ranks of this rank's group."""
        if inter_host:
            first = rank - rank % sharding_group_size

            def to_global(r: int) -> int:
                return first + r
        else:
            first = rank % step

            def to_global(r: int) -> int:
                return first + r * step

        for module_plan in plan.plan.values():
            if not isinstance(module_plan, dict):
                continue
            for ps in module_plan.values():
                if ps.ranks is not None:
                    ps.ranks = [to_global(r) for r in ps.ranks]
                for shard in getattr(ps.sharding_spec, "shards", None) or []:
                    where = shard.placement
                    shard.placement = torch.distributed._remote_device(f"rank:{to_global(where.rank())}/{where.device()}")

    def _group_sharded_modules(self) -> List[nn.Module]:
        return [m for _, m, sharded in _leaves(self._dmp_wrapped_module) if sharded]

    def _replicated_tensors(self, include_optimizer_state: bool) -> Iterator[torch.Tensor]:
        for m in self._modules_to_sync:
            for lookup in getattr(m, "_lookups", []):
                lookup = lookup.module if isinstance(lookup, DistributedDataParallel) else lookup
                for emb in getattr(lookup, "emb_modules", []):
                    tbe = emb.emb_module
                    yield tbe.weights.detach()
                    if include_optimizer_state:
                        yield from (t for t in (tbe.momentum1, tbe.momentum2) if t.numel())

    def sync(self, include_optimizer_state: bool = True) -> None:
        """All-reduce (average) embedding weights and optimizer row/element state over the replica group."""
        assert self._replica_pg is not None, "replica_pg is not initialized!"
        replicas = dist.get_world_size(self._replica_pg)
        with torch.no_grad():
            for t in self._replicated_tensors(include_optimizer_state):
                if self._custom_all_reduce is not None:
                    self._custom_all_reduce([t])
                    continue
                wide = t if t.dtype in (torch.float32, torch.float64) else t.float()
                dist.all_reduce(wide, group=self._replica_pg)
                wide.div_(replicas)
                if wide is not t:
                    t.copy_(wide)

    def set_all_reduce_hook(self, reduce_hook) -> None:
        self._custom_all_reduce = reduce_hook
