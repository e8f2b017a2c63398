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


class DefaultDataParallelWrapper(DataParallelWrapper):
    """DDP over every parameter that is not owned by a sharded module.

    25 MB buckets, static graph, gradients as bucket views; optional fp16 / bf16 gradient compression.
    """

    def __init__(self, bucket_cap_mb: int = 25, static_graph: bool = True, find_unused_parameters: bool = False,
                 allreduce_comm_precision: Optional[str] = None, params_to_ignore: Optional[List[str]] = None,
                 ddp_kwargs: Optional[Dict[str, Any]] = None) -> None:
        self._bucket_cap_mb = bucket_cap_mb
        self._static_graph = static_graph
        self._find_unused_parameters = find_unused_parameters
        self._allreduce_comm_precision = allreduce_comm_precision
        self._additional_params_to_ignore: Set[str] = set(params_to_ignore or [])
        self._ddp_kwargs: Dict[str, Any] = ddp_kwargs or {}

    def _ddp_wrap(self, dmp: "DistributedModelParallel", env: ShardingEnv, device: torch.device, ddp_ignore_param_names: Set[str]) -> None:
        pg = env.process_group
        if pg is None:
            raise RuntimeError("Can only init DDP for ProcessGroup-based ShardingEnv")
        # parameters that take no gradient (slot tables of collision modules) need no all-reduce either
        all_parameter_names = {n for n, p in dmp.named_parameters() if p.requires_grad}
        if len(all_parameter_names - ddp_ignore_param_names) == 0:
            return
        DistributedDataParallel._set_params_and_buffers_to_ignore_for_model(module=dmp._dmp_wrapped_module, params_and_buffers_to_ignore=ddp_ignore_param_names)
        dmp._dmp_wrapped_module = cast(
            nn.Module,
            DistributedDataParallel(
                module=dmp._dmp_wrapped_module.to(device), device_ids=None if device.type == "cpu" else [device], process_group=pg,
                gradient_as_bucket_view=True, broadcast_buffers=False, static_graph=self._static_graph,
                find_unused_parameters=self._find_unused_parameters, bucket_cap_mb=self._bucket_cap_mb, **self._ddp_kwargs,
            ),
        )
        if self._allreduce_comm_precision == "fp16":
            dmp._dmp_wrapped_module.register_comm_hook(None, ddp_default_hooks.fp16_compress_hook)
        elif self._allreduce_comm_precision == "bf16":
            dmp._dmp_wrapped_module.register_comm_hook(None, ddp_default_hooks.bf16_compress_hook)

    def wrap(self, dmp: "DistributedModelParallel", env: ShardingEnv, device: torch.device) -> None:
        if isinstance(dmp._dmp_wrapped_module, DistributedDataParallel):
            return
        sharded_parameter_names = set(DistributedModelParallel._sharded_parameter_names(dmp._dmp_wrapped_module))
        self._ddp_wrap(dmp, env, device, sharded_parameter_names.union(self._additional_params_to_ignore))


def get_unwrapped_module(module: nn.Module) -> nn.Module:
    """Strip ``DistributedModelParallel`` / DDP wrappers."""
    while isinstance(module, DistributedModelParallel) or isinstance(module, DistributedDataParallel):
        if isinstance(module, DistributedModelParallel):
            module = module._dmp_wrapped_module
        else:
            module = module.module
    return module


def get_module(module: nn.Module) -> nn.Module:
    """Strip ``DistributedModelParallel`` wrappers only (data-parallel wrappers stay)."""
    while isinstance(module, DistributedModelParallel):
        module = module._dmp_wrapped_module
    return module


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
        if env is None:
            pg = dist.GroupMember.WORLD
            assert pg is not None, "Process group is not initialized"
            env = ShardingEnv.from_process_group(pg)
        self._env: ShardingEnv = env
        if device is None:
            device = torch.device("cpu")
        self.device: torch.device = device
        if sharders is None:
            sharders = get_default_sharders()
        self._sharder_map: Dict[Type[nn.Module], ModuleSharder[nn.Module]] = {s.module_type: s for s in sharders}
        if data_parallel_wrapper is None:
            data_parallel_wrapper = DefaultDataParallelWrapper()
        self._data_parallel_wrapper: DataParallelWrapper = data_parallel_wrapper
        if plan is None:
            from torchrec_b200.distributed.planner import EmbeddingShardingPlanner, Topology

            planner = EmbeddingShardingPlanner(
                topology=Topology(local_world_size=get_local_size(self._env.world_size), world_size=self._env.world_size, compute_device=self.device.type)
            )
            pg = self._env.process_group
            plan = planner.collective_plan(module, sharders, pg) if pg is not None else planner.plan(module, sharders)
        self._plan: ShardingPlan = plan
        self._dmp_wrapped_module: nn.Module = self._init_dmp(module)
        self._optim: CombinedOptimizer = self._init_optim(self._dmp_wrapped_module)
        if init_parameters:
            self._init_parameters(self.module)
        if init_data_parallel:
            self.init_data_parallel()
        self.model_delta_tracker = self._init_delta_tracker(model_tracker_config, self._dmp_wrapped_module) if model_tracker_config is not None else None

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
        if not self._ddp_wrapped:
            self._data_parallel_wrapper.wrap(self, self._env, self.device)
            self._ddp_wrapped = True

    def copy(self, device: torch.device) -> "DistributedModelParallel":
        """Copy of the wrapper whose dense part lives on ``device``; sharded modules are shared."""
        assert isinstance(device, torch.device)
        with sharded_model_copy(device=None):
            copy_dmp = copy.deepcopy(self)
        copy_dmp_wrapped_module = copy_to_device(self._dmp_wrapped_module, self.device, device)
        copy_dmp._dmp_wrapped_module = copy_dmp_wrapped_module
        return copy_dmp

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
        if isinstance(module, FusedOptimizerModule):
            fused_optims.append((path, module.fused_optimizer))
            return fused_optims
        for name, child in module.named_children():
            self._fused_optim_impl(child, fused_optims, path + "." + name if path else name)
        return fused_optims

    def _shard_modules_impl(self, module: nn.Module, path: str = "") -> nn.Module:
        if isinstance(module, ShardedModule):
            return module
        module_sharding_plan = self._plan.get_plan_for_module(path)
        if module_sharding_plan:
            sharder_key = type(module)
            module = self._sharder_map[sharder_key].shard(module, module_sharding_plan, self._env, self.device, path)
            torch._C._log_api_usage_once(f"torchrec.distributed.{type(module).__name__}")
            return module
        for name, child in module.named_children():
            child = self._shard_modules_impl(child, path + "." + name if path else name)
            setattr(module, name, child)
        return module

    def _init_parameters(self, module: nn.Module) -> None:
        @torch.no_grad()
        def init(m: nn.Module) -> None:
            if isinstance(m, ShardedModule):
                return
            init_parameters(m, self.device)

        module.apply(init)

    # ---- named members with DDP prefixes removed and sharded modules reported under unsharded names ----
    def sparse_grad_parameter_names(self, destination: Optional[List[str]] = None, prefix: str = "") -> List[str]:
        destination = [] if destination is None else destination
        return self._sparse_grad_parameter_names(self.module, destination, prefix)

    def _sparse_grad_parameter_names(self, module: nn.Module, destination: List[str], prefix: str = "") -> List[str]:
        module = get_unwrapped_module(module)
        if isinstance(module, ShardedModule):
            pass
        elif isinstance(module, nn.Embedding):
            if module.sparse:
                destination.append(append_prefix(prefix, "weight"))
        elif isinstance(module, nn.EmbeddingBag):
            if module.sparse:
                destination.append(append_prefix(prefix, "weight"))
        else:
            for name, child in module.named_children():
                self._sparse_grad_parameter_names(child, destination, append_prefix(prefix, name))
        return destination

    def state_dict(self, destination: Optional[Dict[str, Any]] = None, prefix: str = "", keep_vars: bool = False) -> Dict[str, Any]:
        state_dict = get_module(self).state_dict(destination=destination, prefix=prefix, keep_vars=keep_vars)
        torch.nn.modules.utils.consume_prefix_in_state_dict_if_present(state_dict, prefix + _DDP_STATE_DICT_PREFIX)
        add_prefix_to_state_dict(state_dict, prefix)
        return state_dict

    def load_state_dict(self, state_dict: "OrderedDict[str, torch.Tensor]", prefix: str = "", strict: bool = True) -> _IncompatibleKeys:
        return self._load_state_dict(self, state_dict, prefix, strict)

    def _load_state_dict(self, module: nn.Module, state_dict: "OrderedDict[str, torch.Tensor]", prefix: str = "", strict: bool = True) -> _IncompatibleKeys:
        missing_keys: List[str] = []
        unexpected_keys: List[str] = []
        module = get_module(module)
        if isinstance(module, DistributedDataParallel):
            torch.nn.modules.utils.consume_prefix_in_state_dict_if_present(state_dict, prefix)
            add_prefix_to_state_dict(state_dict, prefix + _DDP_STATE_DICT_PREFIX)
        if getattr(module, "_FORCE_STATE_DICT_LOAD", False):
            return module.load_state_dict(state_dict, strict=strict)
        module._load_from_state_dict(state_dict, prefix, {}, strict, missing_keys, unexpected_keys, [])
        for name, child in module.named_children():
            m_keys, u_keys = self._load_state_dict(child, filter_state_dict(state_dict, prefix + name), "", strict)
            missing_keys.extend(m_keys)
            unexpected_keys.extend(u_keys)
        return _IncompatibleKeys(missing_keys=missing_keys, unexpected_keys=unexpected_keys)

    def _named_parameters(self, module: nn.Module, prefix: str = "", recurse: bool = True, strip_ddp: bool = True) -> Iterator[Tuple[str, torch.nn.Parameter]]:
        if strip_ddp:
            module = get_unwrapped_module(module)
        if isinstance(module, ShardedModule):
            yield from module.named_parameters(prefix, recurse)
        else:
            yield from module.named_parameters(prefix, recurse=False)
            for name, child in module.named_children():
                yield from self._named_parameters(child, append_prefix(prefix, name), recurse, strip_ddp)

    def named_parameters(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True) -> Iterator[Tuple[str, torch.nn.Parameter]]:
        gen = self._named_parameters(self.module, prefix, recurse)
        memo = set()
        for key, param in gen:
            if param in memo:
                continue
            if remove_duplicate:
                memo.add(param)
            yield key, param

    def bare_named_parameters(self, prefix: str = "", recurse: bool = True) -> Iterator[Tuple[str, torch.nn.Parameter]]:
        gen = self._named_parameters(self.module, prefix, recurse)
        memo = set()
        for key, param in gen:
            if param in memo:
                continue
            memo.add(param)
            yield key, param

    @staticmethod
    def _sharded_parameter_names(module: nn.Module, prefix: str = "") -> Iterator[str]:
        module = get_unwrapped_module(module)
        if isinstance(module, ShardedModule):
            yield from module.sharded_parameter_names(prefix)
        else:
            for name, child in module.named_children():
                yield from DistributedModelParallel._sharded_parameter_names(child, append_prefix(prefix, name))

    def _named_buffers(self, module: nn.Module, prefix: str = "", recurse: bool = True) -> Iterator[Tuple[str, torch.Tensor]]:
        module = get_unwrapped_module(module)
        if isinstance(module, ShardedModule):
            yield from module.named_buffers(prefix, recurse)
        else:
            yield from module.named_buffers(prefix, recurse=False)
            for name, child in module.named_children():
                yield from self._named_buffers(child, append_prefix(prefix, name), recurse)

    def named_buffers(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True) -> Iterator[Tuple[str, torch.Tensor]]:
        gen = self._named_buffers(self.module, prefix, recurse)
        memo = set()
        for key, param in gen:
            if param in memo:
                continue
            if remove_duplicate:
                memo.add(param)
            yield key, param

    @property
    def fused_optimizer(self) -> KeyedOptimizer:
        return self._optim

    @property
    def plan(self) -> ShardingPlan:
        return self._plan

    @staticmethod
    def _reset_parameters(module: nn.Module) -> None:
        for _, m in module.named_modules():
            if hasattr(m, "reset_parameters"):
                m.reset_parameters()

    def reshard(self, sharded_module_fqn: str, changed_shard_to_params: Dict[str, ParameterSharding]) -> None:
        """Move the shards of ``sharded_module_fqn`` to a new placement at run time (dynamic resharding)."""
        from torchrec_b200.distributed.sharding.dynamic_sharding import reshard_module

        steps = sharded_module_fqn.split(".")
        sharded_module = self.module
        for s in steps:
            sharded_module = getattr(sharded_module, s)
        assert isinstance(sharded_module, ShardedModule)
        reshard_module(self, sharded_module_fqn, sharded_module, changed_shard_to_params)
        self._optim = self._init_optim(self._dmp_wrapped_module)
        self._plan.plan[sharded_module_fqn] = sharded_module.module_sharding_plan


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
        self._global_pg = global_pg
        self._global_rank = dist.get_rank(global_pg)
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
        """``sharding_pg``: ranks that shard together; ``replica_pg``: ranks holding the same shard."""
        rank = dist.get_rank(global_pg)
        backend = dist.get_backend(global_pg)
        n_groups = world_size // sharding_group_size
        sharding_pg = replica_pg = None
        if inter_host:
            shard_groups = [list(range(g * sharding_group_size, (g + 1) * sharding_group_size)) for g in range(n_groups)]
            replica_groups = [list(range(i, world_size, sharding_group_size)) for i in range(sharding_group_size)]
        else:
            shard_groups = [list(range(g, world_size, n_groups)) for g in range(n_groups)]
            replica_groups = [list(range(i * n_groups, (i + 1) * n_groups)) for i in range(sharding_group_size)]
        for ranks in shard_groups:
            pg = dist.new_group(ranks=ranks, backend=backend)
            if rank in ranks:
                sharding_pg = pg
        for ranks in replica_groups:
            pg = dist.new_group(ranks=ranks, backend=backend)
            if rank in ranks:
                replica_pg = pg
        return sharding_pg, replica_pg

    @staticmethod
    def _remap_sharding_plan(plan: ShardingPlan, rank: int, step: int, inter_host: bool, sharding_group_size: int) -> None:
        """Plans are written for ranks ``0..group_size-1``; map them to the global ranks of this rank's group."""
        group_start = (rank // sharding_group_size) * sharding_group_size if inter_host else rank % step
        for _, module_plan in plan.plan.items():
            if not isinstance(module_plan, dict):
                continue
            for _, ps in module_plan.items():
                if ps.ranks is not None:
                    ps.ranks = [r + group_start if inter_host else r * step + group_start for r in ps.ranks]
                if ps.sharding_spec is not None and hasattr(ps.sharding_spec, "shards"):
                    for i, shard in enumerate(ps.sharding_spec.shards):
                        pl = shard.placement
                        r = pl.rank()
                        new_r = r + group_start if inter_host else r * step + group_start
                        dev = pl.device()
                        shard.placement = torch.distributed._remote_device(f"rank:{new_r}/{dev}")

    def _group_sharded_modules(self) -> List[nn.Module]:
        out: List[nn.Module] = []

        def walk(m: nn.Module) -> None:
            if isinstance(m, ShardedModule):
                out.append(m)
                return
            for c in m.children():
                walk(c)

        walk(self._dmp_wrapped_module)
        return out

    def sync(self, include_optimizer_state: bool = True) -> None:
        """All-reduce (average) embedding weights and optimizer row/element state over the replica group."""
        assert self._replica_pg is not None, "replica_pg is not initialized!"
        tensors: List[torch.Tensor] = []
        for m in self._modules_to_sync:
            for lookup in getattr(m, "_lookups", []):
                lk = lookup.module if isinstance(lookup, DistributedDataParallel) else lookup
                for emb in getattr(lk, "emb_modules", []):
                    tbe = emb.emb_module
                    tensors.append(tbe.weights.detach())
                    if include_optimizer_state:
                        if tbe.momentum1.numel():
                            tensors.append(tbe.momentum1)
                        if tbe.momentum2.numel():
                            tensors.append(tbe.momentum2)
        n = dist.get_world_size(self._replica_pg)
        with torch.no_grad():
            for t in tensors:
                if self._custom_all_reduce is not None:
                    self._custom_all_reduce([t])
                else:
                    work = t.float() if t.dtype not in (torch.float32, torch.float64) else t
                    dist.all_reduce(work, group=self._replica_pg)
                    work.div_(n)
                    if work is not t:
                        t.copy_(work)

    def set_all_reduce_hook(self, reduce_hook) -> None:
        self._custom_all_reduce = reduce_hook
