"""Dynamic resharding on gloo: after moving one table to another rank and turning another from table-wise into row-wise,
training continues exactly like an untouched replica (weights AND row-wise Adagrad state moved)
(cf. ``torchrec/distributed/tests/test_dynamic_sharding.py``)."""
import torch

import test_sharding_gloo as T
from torchrec_b200.test_utils.multi_process import MultiProcessContext, run_multi_process


def _worker(rank, world_size):
    from torchrec_b200.distributed import sharding_plan as sp
    from torchrec_b200.distributed.embeddingbag import EmbeddingBagCollectionSharder
    from torchrec_b200.distributed.model_parallel import DistributedModelParallel
    from torchrec_b200.distributed.types import ShardingEnv, ShardingPlan
    from torchrec_b200.modules.embedding_configs import PoolingType
    from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward
    from torchrec_b200.optim.rowwise_adagrad import RowWiseAdagrad

    with MultiProcessContext(rank, world_size, "gloo") as ctx:
        def build():
            torch.manual_seed(0)
            m = T._Model(T._make_ebc(PoolingType.SUM))
            apply_optimizer_in_backward(RowWiseAdagrad, m.ebc.parameters(), {"lr": 0.1, "eps": 1e-8})
            return m

        def dmp_of(m):
            plan = ShardingPlan({"ebc": T._plan_for(m.ebc, "tw", world_size)})
            return DistributedModelParallel(m, env=ShardingEnv.from_process_group(ctx.pg), device=torch.device("cpu"), plan=plan)

        ref, mov = dmp_of(build()), dmp_of(build())
        kjt = T._make_kjt(6, 100 + rank)

        def step(d):
            p, _ = d(kjt)
            p.mean().backward()
            return p.detach()

        torch.testing.assert_close(step(mov), step(ref))
        new = sp.construct_module_sharding_plan(build().ebc, {"t0": sp.table_wise(rank=1), "t1": sp.row_wise(), "t2": sp.table_wise(rank=0), "t3": sp.table_wise(rank=1)},
                                                sharder=EmbeddingBagCollectionSharder(), world_size=world_size, local_size=world_size, device_type="cpu")
        from torchrec_b200.distributed.sharding.dynamic_sharding import output_sharding_plan_delta_single, output_sharding_plans_delta

        volume, delta = output_sharding_plan_delta_single(mov.module.ebc.module_sharding_plan, new, return_data_volume=True)
        assert set(delta) == {"t0", "t1"} and volume > 0  # t2 and t3 stay where they are
        assert set(output_sharding_plans_delta({"ebc": mov.module.ebc.module_sharding_plan}, {"ebc": new})["ebc"][1]) == {"t0", "t1"}
        mov.reshard("ebc", delta)
        assert {k: v.sharding_type for k, v in mov.module.ebc.module_sharding_plan.items()} == {"t0": "table_wise", "t1": "row_wise", "t2": "table_wise", "t3": "table_wise"}
        assert mov.module.ebc.module_sharding_plan["t0"].ranks == [1]
        for _ in range(3):
            torch.testing.assert_close(step(mov), step(ref), rtol=1e-5, atol=1e-6)
        # the DMP-level fused optimizer was rebuilt over the new shards
        assert any("t1" in k for k in mov.fused_optimizer.state_dict()["state"].keys())


def test_reshard_keeps_training_identical():
    run_multi_process(_worker, world_size=2)


def test_plan_update_and_host_offload_helpers():
    from types import SimpleNamespace

    from torchrec_b200.distributed.sharding.dynamic_sharding import move_sharded_tensors_to_cpu, update_module_sharding_plan
    from torchrec_b200.distributed.types import ParameterSharding

    old = ParameterSharding(sharding_type="table_wise", compute_kernel="fused", ranks=[0])
    new = ParameterSharding(sharding_type="table_wise", compute_kernel="fused", ranks=[1])
    info = SimpleNamespace(embedding_config=SimpleNamespace(name="t0"), param_sharding=old)
    other = SimpleNamespace(embedding_config=SimpleNamespace(name="t1"), param_sharding=old)
    module = SimpleNamespace(module_sharding_plan={"t0": old, "t1": old})
    update_module_sharding_plan(module, {"t0": new}, {"table_wise": [info, other]})
    assert module.module_sharding_plan["t0"] is new and info.param_sharding is new and other.param_sharding is old
    try:
        update_module_sharding_plan(SimpleNamespace(), {"t0": new}, {})
        raise AssertionError("a module without a plan must be refused")
    except RuntimeError:
        pass
    nested = {"a": [torch.ones(2), ("x", 3)], "b": {"c": 1.5}}
    out = move_sharded_tensors_to_cpu(nested)
    assert out["b"]["c"] == 1.5 and out["a"][1] == ("x", 3) and torch.equal(out["a"][0], torch.ones(2))
