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
        mov.reshard("ebc", {k: new[k] for k in ("t0", "t1")})
        assert {k: v.sharding_type for k, v in mov.module.ebc.module_sharding_plan.items()} == {"t0": "table_wise", "t1": "row_wise", "t2": "table_wise", "t3": "table_wise"}
        assert mov.module.ebc.module_sharding_plan["t0"].ranks == [1]
        for _ in range(3):
            torch.testing.assert_close(step(mov), step(ref), rtol=1e-5, atol=1e-6)
        # the DMP-level fused optimizer was rebuilt over the new shards
        assert any("t1" in k for k in mov.fused_optimizer.state_dict()["state"].keys())


def test_reshard_keeps_training_identical():
    run_multi_process(_worker, world_size=2)
