"""Composable sharding API: shard one module (or all shardable modules of a model) in place without the
``DistributedModelParallel`` wrapper (``torchrec/distributed/shard.py:40,149``)."""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Type, Union

import torch
import torch.distributed as dist
from torch import nn

from torchrec_b200.distributed.comm import get_local_size
from torchrec_b200.distributed.sharding_plan import get_default_sharders, get_module_to_default_sharders
from torchrec_b200.distributed.types import (
    EmbeddingModuleShardingPlan, ModuleSharder, ParameterSharding, ShardedModule, ShardingEnv, ShardingPlan,
)

ParameterShardingGenerator = Callable[..., ParameterSharding]


def _join_module_path(path: str, name: str) -> str:
    return (path + "." + name) if path else name


def shard(module: nn.Module, plan: Union[EmbeddingModuleShardingPlan, Dict[str, Union[ParameterShardingGenerator, ParameterSharding]]],
          env: Optional[Union[ShardingEnv, dist.ProcessGroup]] = None, device: Optional[torch.device] = None, sharder: Optional[ModuleSharder[nn.Module]] = None) -> nn.Module:
    """Shard ``module`` according to ``plan`` (a module plan, or table -> generator / ParameterSharding) and return the sharded module."""
    torch._C._log_api_usage_once("torchrec_b200.distributed.shard")
    if sharder is None:
        sharder = get_module_to_default_sharders().get(type(module), None)
    assert sharder is not None, f"Could not find a valid sharder type for {type(module)}"
    if env is None:
        pg = dist.distributed_c10d._get_default_group()
        env = ShardingEnv.from_process_group(pg)
    elif isinstance(env, dist.ProcessGroup):
        env = ShardingEnv.from_process_group(env)
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    if not isinstance(plan, EmbeddingModuleShardingPlan) and any(callable(v) for v in plan.values()):
        from torchrec_b200.distributed.sharding_plan import construct_module_sharding_plan

        plan = construct_module_sharding_plan(module, plan, sharder=sharder, local_size=get_local_size(env.world_size), world_size=env.world_size, device_type=device.type)
    return sharder.shard(module, plan, env, device)


def shard_modules(module: nn.Module, env: Optional[Union[ShardingEnv, dist.ProcessGroup]] = None, device: Optional[torch.device] = None,
                  plan: Optional[ShardingPlan] = None, sharders: Optional[List[ModuleSharder[nn.Module]]] = None, init_params: bool = False) -> nn.Module:
    """Replace every shardable submodule of ``module`` by its sharded form in place (plans with the default planner when no plan is given)."""
    torch._C._log_api_usage_once("torchrec_b200.distributed.shard_modules")
    if sharders is None:
        sharders = get_default_sharders()
    if env is None:
        env = ShardingEnv.from_process_group(dist.distributed_c10d._get_default_group())
    elif isinstance(env, dist.ProcessGroup):
        env = ShardingEnv.from_process_group(env)
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    sharder_map: Dict[Type[nn.Module], ModuleSharder[nn.Module]] = {s.module_type: s for s in sharders}
    if plan is None:
        from torchrec_b200.distributed.planner import EmbeddingShardingPlanner, Topology

        planner = EmbeddingShardingPlanner(topology=Topology(local_world_size=get_local_size(env.world_size), world_size=env.world_size, compute_device=device.type))
        pg = env.process_group
        plan = planner.collective_plan(module, sharders, pg) if pg is not None else planner.plan(module, sharders)
    if type(module) in sharder_map and "" in plan.plan:
        return sharder_map[type(module)].shard(module, plan.get_plan_for_module(""), env, device)

    def replace(m: nn.Module, path: str) -> None:
        for name, child in list(m.named_children()):
            child_path = _join_module_path(path, name)
            if isinstance(child, ShardedModule):
                continue
            sub_plan = plan.get_plan_for_module(child_path)
            if sub_plan is not None and type(child) in sharder_map:
                setattr(m, name, sharder_map[type(child)].shard(child, sub_plan, env, device, child_path))
            else:
                replace(child, child_path)

    replace(module, "")
    if init_params:
        for m in module.modules():
            if not isinstance(m, ShardedModule) and hasattr(m, "reset_parameters") and any(p.device.type == "meta" for p in m.parameters(recurse=False)):
                m.to_empty(device=device, recurse=False)
                m.reset_parameters()
    return module
