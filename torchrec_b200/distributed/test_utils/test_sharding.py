"""Harness: train one step of a model sharded by the planner and of its unsharded twin on the same data, compare predictions.

``sharding_single_rank_test`` is the body of one rank (launch it with ``run_multi_process``).  The unsharded model sees the
global batch, every rank of the sharded model its slice; after one optimizer step on both, the second forward's predictions of
all ranks, gathered, must equal the global model's.  Counterpart of ``torchrec/distributed/test_utils/test_sharding.py:760-1037``."""
from __future__ import annotations

import copy
from typing import Any, Dict, List, Optional, Sequence, Type

import torch
import torch.distributed as dist
from torch import nn

from torchrec_b200.distributed.model_parallel import DistributedModelParallel
from torchrec_b200.distributed.planner import EmbeddingShardingPlanner, ParameterConstraints, Topology
from torchrec_b200.distributed.test_utils.test_model import ModelInput, TestSparseNN
from torchrec_b200.distributed.types import ModuleSharder, ShardingEnv
from torchrec_b200.modules.embedding_configs import BaseEmbeddingConfig
from torchrec_b200.test_utils.multi_process import MultiProcessContext


def create_test_sharder(sharder_type: str, sharding_type: str, kernel_type: str, fused_params: Optional[Dict[str, Any]] = None,
                        qcomm_codecs_registry=None) -> ModuleSharder[nn.Module]:
    """``sharder_type``: ``"embedding_bag_collection"`` or ``"embedding_collection"``."""
    from torchrec_b200.distributed.test_utils.test_model import TestEBCSharder, TestECSharder

    table = {"embedding_bag_collection": TestEBCSharder, "embedding_collection": TestECSharder}
    if sharder_type not in table:
        raise ValueError(f"Sharder not supported {sharder_type}")
    return table[sharder_type](sharding_type, kernel_type, fused_params, qcomm_codecs_registry)


def generate_inputs(world_size: int, tables: Sequence[BaseEmbeddingConfig], weighted_tables: Optional[Sequence[BaseEmbeddingConfig]] = None,
                    batch_size: int = 4, num_float_features: int = 16, seed: int = 0):
    return ModelInput.generate(batch_size=batch_size, world_size=world_size, num_float_features=num_float_features, tables=tables,
                               weighted_tables=weighted_tables or [], pooling_avg=3, random_seed=seed)


def gen_model_and_input(model_class: Type[nn.Module], tables, weighted_tables, world_size: int, num_float_features: int = 16,
                        batch_size: int = 4, seed: int = 0, **model_kwargs):
    torch.manual_seed(seed)
    model = model_class(tables=tables, num_float_features=num_float_features, weighted_tables=weighted_tables, **model_kwargs)
    return model, [generate_inputs(world_size, tables, weighted_tables, batch_size, num_float_features, seed)]


def sharding_single_rank_test(rank: int, world_size: int, tables: List[BaseEmbeddingConfig], sharders: List[ModuleSharder[nn.Module]],
                              backend: str = "gloo", model_class: Type[nn.Module] = TestSparseNN,
                              weighted_tables: Optional[List[BaseEmbeddingConfig]] = None,
                              constraints: Optional[Dict[str, ParameterConstraints]] = None, local_size: Optional[int] = None,
                              lr: float = 0.1, rtol: float = 1e-4, atol: float = 1e-5) -> None:
    with MultiProcessContext(rank, world_size, backend, local_size) as ctx:
        device = ctx.device if hasattr(ctx, "device") else torch.device("cpu")
        global_model, inputs = gen_model_and_input(model_class, tables, weighted_tables, world_size)
        global_input, local_inputs = inputs[0]
        local_model = copy.deepcopy(global_model)
        global_model = global_model.to(device)
        planner = EmbeddingShardingPlanner(topology=Topology(world_size=world_size, local_world_size=local_size or world_size, compute_device=device.type),
                                           constraints=constraints, batch_size=local_inputs[0].float_features.shape[0])
        plan = planner.collective_plan(local_model, sharders, ctx.pg)
        dmp = DistributedModelParallel(local_model, env=ShardingEnv.from_process_group(ctx.pg), plan=plan, sharders=sharders, device=device)
        dmp.load_state_dict(copy.deepcopy(global_model.state_dict()))
        fused = getattr(dmp, "fused_optimizer", None)
        fused_names = set(fused.params.keys()) if fused is not None and hasattr(fused, "params") else set()
        dense_opt = torch.optim.SGD([p for n, p in dmp.named_parameters() if n not in fused_names and p.requires_grad], lr=lr)
        global_opt = torch.optim.SGD(global_model.parameters(), lr=lr)
        mine = local_inputs[rank].to(device)
        whole = global_input.to(device)

        # one step on each
        global_opt.zero_grad()
        g_loss, _ = global_model(whole)
        g_loss.backward()
        global_opt.step()
        dense_opt.zero_grad()
        l_loss, _ = dmp(mine)
        # the global loss is a mean over world_size times as many samples: DDP averages the dense gradients over ranks and the
        # embedding exchanges divide theirs by the world size, so both steps agree
        l_loss.backward()
        dense_opt.step()

        global_model.eval()
        dmp.eval()
        with torch.no_grad():
            g_pred = global_model(whole)
            l_pred = dmp(mine)
        gathered = [torch.empty_like(l_pred) for _ in range(world_size)]
        dist.all_gather(gathered, l_pred.contiguous(), group=ctx.pg)
        torch.testing.assert_close(torch.cat(gathered).cpu(), g_pred.cpu(), rtol=rtol, atol=atol)
