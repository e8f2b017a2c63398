"""2D parallelism on four gloo ranks: two sharding groups of two ranks; tables are sharded inside a group and the groups are
replicas whose weights and optimizer state ``sync()`` averages (cf. ``torchrec/distributed/tests/test_2d_sharding.py``)."""
import copy

import pytest
import torch
import torch.distributed as dist

import test_sharding_gloo as T
from torchrec_b200.test_utils.multi_process import MultiProcessContext, run_multi_process


def _run(rank, world_size, inter_host):
    from torchrec_b200.distributed.model_parallel import DMPCollection
    from torchrec_b200.distributed.types import ShardingPlan
    from torchrec_b200.modules.embedding_configs import PoolingType
    from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward
    from torchrec_b200.optim.rowwise_adagrad import RowWiseAdagrad

    with MultiProcessContext(rank, world_size, "gloo", timeout_s=120) as ctx:
        torch.manual_seed(0)
        group_size = 2
        model = T._Model(T._make_ebc(PoolingType.SUM))
        reference = copy.deepcopy(model)
        apply_optimizer_in_backward(RowWiseAdagrad, model.ebc.parameters(), {"lr": 0.1, "eps": 1e-8})
        plan = ShardingPlan({"ebc": T._plan_for(model.ebc, "mixed", group_size)})  # written for ranks 0..1 of one group
        dmp = DMPCollection(model, device=torch.device("cpu"), plan=plan, world_size=world_size, sharding_group_size=group_size, global_pg=ctx.pg,
                            use_inter_host_allreduce=inter_host)
        dmp.load_state_dict(copy.deepcopy(reference.state_dict()))
        shard_ranks = dist.get_process_group_ranks(dmp._sharding_pg)
        replica_ranks = dist.get_process_group_ranks(dmp._replica_pg)
        assert len(shard_ranks) == 2 and len(replica_ranks) == 2 and rank in shard_ranks and rank in replica_ranks
        assert set(shard_ranks) & set(replica_ranks) == {rank}
        if inter_host:
            assert shard_ranks == [0, 1] or shard_ranks == [2, 3]
        else:
            assert shard_ranks == [0, 2] or shard_ranks == [1, 3]
        # every table shard sits on a rank of this rank's group
        for name, ps in plan.plan["ebc"].items():
            assert set(ps.ranks) <= set(shard_ranks), (name, ps.ranks, shard_ranks)
        dense_params = [p for n, p in dmp.named_parameters() if "ebc" not in n]
        opt = torch.optim.SGD(dense_params, lr=0.1)
        # replicas see different batches, so their tables drift apart ...
        for step in range(2):
            opt.zero_grad()
            pred, _ = dmp(T._make_kjt(6, 500 + 10 * step + rank))
            pred.mean().backward()
            opt.step()
        tbes = [emb.emb_module for m in dmp._modules_to_sync for lk in m._lookups for emb in getattr(lk.module if hasattr(lk, "module") else lk, "emb_modules", [])]
        assert tbes
        peer = [r for r in replica_ranks if r != rank][0]

        def replica_gap():
            gaps = []
            for t in tbes:
                mine = t.weights.detach().clone()
                both = [torch.empty_like(mine) for _ in range(2)]
                dist.all_gather(both, mine, group=dmp._replica_pg)
                gaps.append(float((both[0] - both[1]).abs().max()))
            return max(gaps)

        assert replica_gap() > 0
        before = [t.weights.detach().clone() for t in tbes]
        dmp.sync()
        # ... and sync() makes them equal again: the mean of the two replicas
        assert replica_gap() == 0
        for t, b in zip(tbes, before):
            both = [torch.empty_like(b) for _ in range(2)]
            dist.all_gather(both, b, group=dmp._replica_pg)
            torch.testing.assert_close(t.weights.detach(), (both[0] + both[1]) / 2)
        # the state dict keeps the unsharded model's keys
        assert set(dmp.state_dict().keys()) == set(reference.state_dict().keys())


@pytest.mark.parametrize("inter_host", [False, True])
def test_dmp_collection_two_groups_of_two(inter_host):
    run_multi_process(_run, world_size=4, inter_host=inter_host, timeout_s=400)
