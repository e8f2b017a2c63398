"""Sharded feature-processed and in-training-pruning collections on CPU/gloo, world size 2."""
import copy

import pytest
import torch
import torch.distributed as dist

import test_sharding_gloo as T
from torchrec_b200.test_utils.multi_process import MultiProcessContext, run_multi_process


class _FPModel(torch.nn.Module):
    def __init__(self, fp_ebc):
        super().__init__()
        self.fp_ebc = fp_ebc
        self.over = torch.nn.Linear(sum(len(f) for _, _, f in T.TABLES) * 16, 1)

    def forward(self, kjt):
        kt = self.fp_ebc(kjt)
        if hasattr(kt, "wait"):
            kt = kt.wait()
        return self.over(kt.values()), kt


def _fp_parity(rank, world_size, sharding, collection):
    from torchrec_b200.distributed.fp_embeddingbag import FeatureProcessedEmbeddingBagCollectionSharder
    from torchrec_b200.distributed.model_parallel import DistributedModelParallel
    from torchrec_b200.distributed.sharding_plan import get_default_sharders
    from torchrec_b200.distributed.types import ShardingEnv, ShardingPlan
    from torchrec_b200.modules.embedding_configs import PoolingType
    from torchrec_b200.modules.feature_processor_ import PositionWeightedModule, PositionWeightedModuleCollection
    from torchrec_b200.modules.fp_embedding_modules import FeatureProcessedEmbeddingBagCollection
    from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    with MultiProcessContext(rank, world_size, "gloo") as ctx:
        torch.manual_seed(0)
        B, lr = 6, 0.1
        feats = [f for _, _, fs in T.TABLES for f in fs]
        if collection:
            fps = PositionWeightedModuleCollection({f: 5 for f in feats})
        else:
            fps = {f: PositionWeightedModule(max_feature_length=5) for f in feats[:3]}
        global_model = _FPModel(FeatureProcessedEmbeddingBagCollection(T._make_ebc(PoolingType.SUM, weighted=True), fps))
        with torch.no_grad():
            for p in global_model.fp_ebc._feature_processors.parameters():
                p.copy_(torch.rand_like(p) + 0.5)
        local_model = copy.deepcopy(global_model)
        apply_optimizer_in_backward(torch.optim.SGD, local_model.fp_ebc._embedding_bag_collection.parameters(), {"lr": lr})
        plan = ShardingPlan({"fp_ebc": T._plan_for(local_model.fp_ebc._embedding_bag_collection, sharding, world_size)})
        dmp = DistributedModelParallel(local_model, env=ShardingEnv.from_process_group(ctx.pg), device=torch.device("cpu"), plan=plan,
                                       sharders=get_default_sharders() + [FeatureProcessedEmbeddingBagCollectionSharder()])
        dmp.load_state_dict(copy.deepcopy(global_model.state_dict()))
        dense_opt = torch.optim.SGD([p for n, p in dmp.named_parameters() if "_embedding_bag_collection" not in n], lr=lr)
        g_opt = torch.optim.SGD(global_model.parameters(), lr=lr)
        kjts = [T._make_kjt(B, 100 + r) for r in range(world_size)]
        keys = kjts[0].keys()
        vals, lens = [], []
        for k in keys:
            for kj in kjts:
                vals.append(kj[k].values()); lens.append(kj[k].lengths())
        global_kjt = KeyedJaggedTensor.from_lengths_sync(keys=keys, values=torch.cat(vals), lengths=torch.cat(lens))
        for step in range(2):
            g_opt.zero_grad()
            g_pred, _ = global_model(global_kjt)
            g_pred.mean().backward()
            g_opt.step()
            dense_opt.zero_grad()
            l_pred, _ = dmp(kjts[rank])
            l_pred.mean().backward()
            dense_opt.step()
            torch.testing.assert_close(l_pred.detach(), g_pred.detach()[rank * B:(rank + 1) * B], rtol=1e-4, atol=1e-5)
        sd = dmp.state_dict()
        for name, gt in global_model.state_dict().items():
            v = sd[name]
            if hasattr(v, "local_shards"):
                mine = torch.zeros_like(gt)
                for s in v.local_shards():
                    ro, co = s.metadata.shard_offsets
                    rs, cs = s.metadata.shard_sizes
                    mine[ro:ro + rs, co:co + cs] = s.tensor
                dist.all_reduce(mine)
                v = mine
            torch.testing.assert_close(v, gt, rtol=1e-4, atol=1e-5, msg=lambda m: f"{name}: {m}")


@pytest.mark.parametrize("sharding,collection", [("tw", True), ("rw", True), ("mixed", True), ("tw", False)])
def test_sharded_fp_ebc_parity(sharding, collection):
    run_multi_process(_fp_parity, world_size=2, sharding=sharding, collection=collection)


def _itep_run(rank, world_size, sharding):
    from torchrec_b200.distributed.itep_embeddingbag import ITEPEmbeddingBagCollectionSharder
    from torchrec_b200.distributed.model_parallel import DistributedModelParallel
    from torchrec_b200.distributed.sharding_plan import get_default_sharders
    from torchrec_b200.distributed.types import ShardingEnv, ShardingPlan
    from torchrec_b200.modules.embedding_configs import PoolingType
    from torchrec_b200.modules.itep_embedding_modules import ITEPEmbeddingBagCollection
    from torchrec_b200.modules.itep_modules import GenericITEPModule
    from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    with MultiProcessContext(rank, world_size, "gloo") as ctx:
        torch.manual_seed(0)
        ebc = T._make_ebc(PoolingType.SUM)
        unpruned = {"t0": 1000, "t2": 330}  # t0 has 100 rows, t2 has 33
        model = torch.nn.Module()
        model.itep = ITEPEmbeddingBagCollection(ebc, GenericITEPModule(unpruned, lookups=None, pruning_interval=5))
        apply_optimizer_in_backward(torch.optim.SGD, ebc.parameters(), {"lr": 0.1})
        plan = ShardingPlan({"itep": T._plan_for(ebc, sharding, world_size)})
        dmp = DistributedModelParallel(model, env=ShardingEnv.from_process_group(ctx.pg), device=torch.device("cpu"), plan=plan,
                                       sharders=get_default_sharders() + [ITEPEmbeddingBagCollectionSharder()])
        sharded = dmp.module.itep
        g = torch.Generator().manual_seed(7 + rank)
        hot = {"f0": 777, "f3": 301}
        for it in range(7):
            keys, lens, vals = [], [], []
            for (r, _, feats) in T.TABLES:
                for f in feats:
                    keys.append(f)
                    l = torch.randint(1, 4, (4,), generator=g)
                    hi = unpruned.get({"f0": "t0", "f3": "t2"}.get(f, ""), r)
                    v = torch.randint(0, hi, (int(l.sum()),), generator=g)
                    if f in hot:
                        v[0] = hot[f]  # an id beyond the pruned size that shows up in every batch
                    lens.append(l); vals.append(v)
            kjt = KeyedJaggedTensor.from_lengths_sync(keys=keys, values=torch.cat(vals), lengths=torch.cat(lens))
            out = sharded(kjt).wait()
            assert out.values().shape == (4, 16 * 5) and torch.isfinite(out.values()).all()
            out.values().sum().backward()
        assert int(sharded._iter) == 7
        sd = dmp.state_dict()
        assert "itep._iter" in sd and any(k.endswith("t0_itp_address_lookup") for k in sd) or sharding == "tw"
        # the hot ids own a row by now on the rank that serves them
        mods = [sharded._itep_module, sharded._rowwise_itep_module]
        owned = 0
        for m in mods:
            for name, idx in m.table_name_to_idx.items():
                lo = m.buffer_offsets_list[idx]
                al = m.address_lookup[lo:m.buffer_offsets_list[idx + 1]]
                size = m.emb_sizes_list[idx]
                assert int((al >= 0).sum()) == size and int(al.clamp(min=0).max()) < size
                hid = hot["f0"] if name == "t0" else hot["f3"]
                if sharding == "rw":
                    block = -(-unpruned[name] // world_size)
                    if hid // block != rank:
                        continue
                    hid = hid % block
                owned += int(al[hid] >= 0)
        total = torch.tensor([owned])
        dist.all_reduce(total)
        assert int(total) == 2, f"hot ids own {int(total)} rows"


@pytest.mark.parametrize("sharding", ["tw", "rw"])
def test_sharded_itep_ebc(sharding):
    run_multi_process(_itep_run, world_size=2, sharding=sharding)
