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


def _mc_models(device):
    from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig
    from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
    from torchrec_b200.modules.hash_mc_modules import HashZchManagedCollisionModule
    from torchrec_b200.modules.mc_embedding_modules import ManagedCollisionEmbeddingBagCollection
    from torchrec_b200.modules.mc_modules import LFU_EvictionPolicy, ManagedCollisionCollection, MCHManagedCollisionModule

    cfgs = [EmbeddingBagConfig(name="t0", embedding_dim=8, num_embeddings=64, feature_names=["f0", "f1"]),
            EmbeddingBagConfig(name="t1", embedding_dim=8, num_embeddings=32, feature_names=["f2"])]
    ebc = EmbeddingBagCollection(tables=cfgs)
    mcc = ManagedCollisionCollection({
        "t0": HashZchManagedCollisionModule(zch_size=64, device=device, total_num_buckets=2, max_probe=32),
        "t1": MCHManagedCollisionModule(zch_size=32, device=device, eviction_policy=LFU_EvictionPolicy(), eviction_interval=2, input_hash_size=4000),
    }, cfgs)
    return ManagedCollisionEmbeddingBagCollection(ebc, mcc, return_remapped_features=True)


def _mc_run(rank, world_size):
    from torchrec_b200.distributed import sharding_plan as sp
    from torchrec_b200.distributed.mc_embeddingbag import ManagedCollisionEmbeddingBagCollectionSharder
    from torchrec_b200.distributed.model_parallel import DistributedModelParallel
    from torchrec_b200.distributed.sharding_plan import get_default_sharders
    from torchrec_b200.distributed.types import ShardingEnv, ShardingPlan
    from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    with MultiProcessContext(rank, world_size, "gloo") as ctx:
        torch.manual_seed(0)
        dev = torch.device("cpu")
        global_model = torch.nn.Module()
        global_model.mc = _mc_models(dev)
        local_model = copy.deepcopy(global_model)
        apply_optimizer_in_backward(torch.optim.SGD, local_model.mc._embedding_module.parameters(), {"lr": 0.1})
        sharder = ManagedCollisionEmbeddingBagCollectionSharder()
        mplan = sp.construct_module_sharding_plan(local_model.mc._embedding_module, {"t0": sp.row_wise(), "t1": sp.row_wise()}, sharder=sharder._e_sharder,
                                                  world_size=world_size, local_size=world_size, device_type="cpu")
        dmp = DistributedModelParallel(local_model, env=ShardingEnv.from_process_group(ctx.pg), device=dev, plan=ShardingPlan({"mc": mplan}),
                                       sharders=get_default_sharders() + [sharder])
        sd = {k: v for k, v in global_model.state_dict().items() if "_embedding_module" in k}
        dmp.load_state_dict(sd, strict=False)
        B = 4
        gen = torch.Generator().manual_seed(11)
        per_rank = []
        for r in range(world_size):
            lens = torch.randint(1, 4, (3 * B,), generator=gen)
            n = int(lens.sum())
            vals = torch.randint(0, 10**9, (n,), generator=gen)
            n2 = int(lens[2 * B:].sum())
            vals[n - n2:] = torch.randint(0, 4000, (n2,), generator=gen)  # the sort-based module has a bounded input space
            per_rank.append((vals, lens))
        mk = lambda v, l: KeyedJaggedTensor.from_lengths_sync(keys=["f0", "f1", "f2"], values=v, lengths=l)
        keys = ["f0", "f1", "f2"]
        gv, gl = [], []
        for k in range(3):
            for v, l in per_rank:
                kj = mk(v, l)[keys[k]]
                gv.append(kj.values()); gl.append(kj.lengths())
        global_kjt = mk(torch.cat(gv), torch.cat(gl))
        g_out, g_remapped = global_model.mc(global_kjt)
        l_out_aw, l_remapped = dmp.module.mc(mk(*per_rank[rank]))
        l_out = l_out_aw.wait()
        # the hash-based table gives the same rows sharded and unsharded -> identical pooled values
        for f in ("f0", "f1"):
            torch.testing.assert_close(l_out[f], g_out[f][rank * B:(rank + 1) * B], rtol=1e-5, atol=1e-6)
        assert l_out["f2"].shape == (B, 8)
        # the remapped ids come back to the rank whose batch they belong to, in the order of its input
        rk = l_remapped.wait()
        mine = mk(*per_rank[rank])
        assert rk.keys() == keys and torch.equal(rk.lengths(), mine.lengths())
        for f in ("f0", "f1"):
            lens = mine[f].lengths()
            g_jt = g_remapped[f]
            g_off = g_jt.offsets()
            want = g_jt.values()[int(g_off[rank * B]):int(g_off[(rank + 1) * B])]
            assert torch.equal(rk[f].values(), want), (f, rk[f].values(), want)
            assert torch.equal(rk[f].lengths(), lens)
        assert ((rk["f2"].values() >= 0) & (rk["f2"].values() < 32)).all()
        l_out.values().sum().backward()
        # checkpoint: slot tables come out as shards of the global table and load back
        full = dmp.state_dict()
        key = "mc._managed_collision_collection._managed_collision_modules.t0._hash_zch_identities"
        assert hasattr(full[key], "local_shards") and tuple(full[key].size()) == (64, 1)
        g_ident = global_model.mc._managed_collision_collection._managed_collision_modules["t0"]._hash_zch_identities
        assert torch.equal(full[key].local_shards()[0].tensor, g_ident[32 * rank:32 * rank + 32])
        dmp.load_state_dict(full)
        dmp.load_state_dict({k: v for k, v in global_model.state_dict().items()}, strict=False)


def test_sharded_mc_ebc():
    run_multi_process(_mc_run, world_size=2)


def _fused_run(rank, world_size):
    from torchrec_b200.distributed import sharding_plan as sp
    from torchrec_b200.distributed.model_parallel import DistributedModelParallel
    from torchrec_b200.distributed.types import ShardingEnv, ShardingPlan
    from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig
    from torchrec_b200.modules.fused_embedding_modules import FusedEmbeddingBagCollection

    with MultiProcessContext(rank, world_size, "gloo") as ctx:
        torch.manual_seed(0)
        cfgs = [EmbeddingBagConfig(name=f"t{i}", num_embeddings=r, embedding_dim=d, feature_names=list(f)) for i, (r, d, f) in enumerate(T.TABLES)]
        g = torch.nn.Module()
        g.ebc = FusedEmbeddingBagCollection(cfgs, torch.optim.SGD, {"lr": 0.1})
        l = torch.nn.Module()
        l.ebc = FusedEmbeddingBagCollection(copy.deepcopy(cfgs), torch.optim.SGD, {"lr": 0.1})
        l.ebc.load_state_dict(g.ebc.state_dict())
        sharders = sp.get_default_sharders()
        fs = next(s for s in sharders if s.module_type is FusedEmbeddingBagCollection)
        gens = {c.name: [sp.table_wise(rank=0), sp.row_wise(), sp.column_wise(ranks=[1, 0]), sp.table_wise(rank=1)][i] for i, c in enumerate(cfgs)}
        mplan = sp.construct_module_sharding_plan(l.ebc, gens, sharder=fs, world_size=world_size, local_size=world_size, device_type="cpu")
        dmp = DistributedModelParallel(l, env=ShardingEnv.from_process_group(ctx.pg), device=torch.device("cpu"), plan=ShardingPlan({"ebc": mplan}), sharders=sharders)
        B = 6
        kjts = [T._make_kjt(B, 100 + r) for r in range(world_size)]
        for step in range(2):
            outs = []
            for r in range(world_size):
                o = g.ebc(kjts[r])
                outs.append(o)
            # the single-device module sees both batches; gradients of a mean over the global batch
            (sum(o.values().sum() for o in outs) / world_size).backward()
            lo = dmp.module.ebc(kjts[rank]).wait()
            torch.testing.assert_close(lo.values(), outs[rank].values().detach(), rtol=1e-5, atol=1e-6)
            lo.values().sum().backward()


def test_sharded_fused_ebc_matches_single_device():
    run_multi_process(_fused_run, world_size=2)


class _TowerInteraction(torch.nn.Module):
    def __init__(self, in_dim):
        super().__init__()
        self.lin = torch.nn.Linear(in_dim, 4)

    def forward(self, kt):
        return torch.relu(self.lin(kt.values()))


def _tower_run(rank, world_size):
    from torchrec_b200.distributed import sharding_plan as sp
    from torchrec_b200.distributed.embedding_tower_sharding import EmbeddingTowerSharder
    from torchrec_b200.distributed.model_parallel import DistributedModelParallel
    from torchrec_b200.distributed.types import ShardingEnv, ShardingPlan
    from torchrec_b200.modules.embedding_configs import PoolingType
    from torchrec_b200.modules.embedding_tower import EmbeddingTower
    from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    with MultiProcessContext(rank, world_size, "gloo") as ctx:
        torch.manual_seed(0)
        B, lr = 6, 0.1
        g = torch.nn.Module()
        g.tower = EmbeddingTower(T._make_ebc(PoolingType.SUM), _TowerInteraction(5 * 16))
        g.head = torch.nn.Linear(4, 1)
        l = copy.deepcopy(g)
        apply_optimizer_in_backward(torch.optim.SGD, l.tower.embedding.parameters(), {"lr": lr})
        sharder = EmbeddingTowerSharder()
        mplan = sp.construct_module_sharding_plan(l.tower.embedding, {f"t{i}": sp.table_wise(rank=1) for i in range(4)}, sharder=sharder._embedding_sharder,
                                                  world_size=world_size, local_size=world_size, device_type="cpu")
        dmp = DistributedModelParallel(l, env=ShardingEnv.from_process_group(ctx.pg), device=torch.device("cpu"), plan=ShardingPlan({"tower": mplan}),
                                       sharders=sp.get_default_sharders() + [sharder])
        dmp.load_state_dict(copy.deepcopy(g.state_dict()))
        assert dmp.module.tower.owner_rank == 1
        dense_params = [p for n, p in dmp.named_parameters() if "embedding" not in n]
        opt = torch.optim.SGD(dense_params, lr=lr)
        g_opt = torch.optim.SGD(g.parameters(), lr=lr)
        kjts = [T._make_kjt(B, 100 + r) for r in range(world_size)]
        keys = kjts[0].keys()
        vals, lens = [], []
        for k in keys:
            for kj in kjts:
                vals.append(kj[k].values()); lens.append(kj[k].lengths())
        global_kjt = KeyedJaggedTensor.from_lengths_sync(keys=keys, values=torch.cat(vals), lengths=torch.cat(lens))
        for step in range(2):
            g_opt.zero_grad()
            g_pred = g.head(g.tower(global_kjt))
            g_pred.mean().backward()
            g_opt.step()
            opt.zero_grad()
            out = dmp.module.tower(kjts[rank]).wait()
            assert out.shape == (B, 4)
            l_pred = dmp.module.head(out)
            l_pred.mean().backward()
            # the head is replicated: average its gradient by hand (the bare submodule call bypasses the wrapper's hooks)
            for p in dmp.module.head.parameters():
                dist.all_reduce(p.grad)
                p.grad /= world_size
            opt.step()
            torch.testing.assert_close(l_pred.detach(), g_pred.detach()[rank * B:(rank + 1) * B], rtol=1e-4, atol=1e-5)
        if rank == 1:  # the interaction was trained where the tower lives
            torch.testing.assert_close(dmp.module.tower.interaction.lin.weight, g.tower.interaction.lin.weight, rtol=1e-4, atol=1e-5)


def _spread_tower_run(rank, world_size, kind):
    """A tower whose tables are spread over the ranks (row-wise / table-row-wise / column-wise): pooled rows arrive at the rank that
    owns the sample, the interaction runs there with replicated parameters, and the whole model matches the unsharded one."""
    from torchrec_b200.distributed import sharding_plan as sp
    from torchrec_b200.distributed.embedding_tower_sharding import EmbeddingTowerSharder
    from torchrec_b200.distributed.model_parallel import DistributedModelParallel
    from torchrec_b200.distributed.types import ShardingEnv, ShardingPlan
    from torchrec_b200.modules.embedding_configs import PoolingType
    from torchrec_b200.modules.embedding_tower import EmbeddingTower
    from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    class Model(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.tower = EmbeddingTower(T._make_ebc(PoolingType.SUM), _TowerInteraction(5 * 16))
            self.head = torch.nn.Linear(4, 1)

        def forward(self, kjt):
            out = self.tower(kjt)
            return self.head(out.wait() if hasattr(out, "wait") else out)

    with MultiProcessContext(rank, world_size, "gloo") as ctx:
        torch.manual_seed(0)
        B, lr = 6, 0.1
        g = Model()
        l = copy.deepcopy(g)
        apply_optimizer_in_backward(torch.optim.SGD, l.tower.embedding.parameters(), {"lr": lr})
        sharder = EmbeddingTowerSharder()
        how = {"row_wise": sp.row_wise(), "table_row_wise": sp.table_row_wise(host_index=0), "column_wise": sp.column_wise(ranks=list(range(world_size)))}[kind]
        mplan = sp.construct_module_sharding_plan(l.tower.embedding, {f"t{i}": how for i in range(4)}, sharder=sharder._embedding_sharder,
                                                  world_size=world_size, local_size=world_size, device_type="cpu")
        dmp = DistributedModelParallel(l, env=ShardingEnv.from_process_group(ctx.pg), device=torch.device("cpu"), plan=ShardingPlan({"tower": mplan}),
                                       sharders=sp.get_default_sharders() + [sharder])
        dmp.load_state_dict(copy.deepcopy(g.state_dict()))
        assert dmp.module.module.tower.owner_rank == -1 if hasattr(dmp.module, "module") else True
        dense_params = [p for n, p in dmp.named_parameters() if "embedding" not in n]
        assert len(dense_params) == 4  # interaction and head, both replicated
        opt = torch.optim.SGD(dense_params, lr=lr)
        g_opt = torch.optim.SGD(g.parameters(), lr=lr)
        kjts = [T._make_kjt(B, 100 + r) for r in range(world_size)]
        keys = kjts[0].keys()
        vals, lens = [], []
        for k in keys:
            for kj in kjts:
                vals.append(kj[k].values()); lens.append(kj[k].lengths())
        global_kjt = KeyedJaggedTensor.from_lengths_sync(keys=keys, values=torch.cat(vals), lengths=torch.cat(lens))
        for step in range(3):
            g_opt.zero_grad()
            g_pred = g(global_kjt)
            g_pred.mean().backward()
            g_opt.step()
            opt.zero_grad()
            l_pred = dmp(kjts[rank])
            l_pred.mean().backward()  # the data-parallel wrapper averages the gradients of the interaction and the head
            opt.step()
            torch.testing.assert_close(l_pred.detach(), g_pred.detach()[rank * B:(rank + 1) * B], rtol=1e-4, atol=1e-5)
        inner = dmp.module.module if hasattr(dmp.module, "module") else dmp.module
        torch.testing.assert_close(inner.tower.interaction.lin.weight.detach(), g.tower.interaction.lin.weight.detach(), rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("kind", ["row_wise", "table_row_wise", "column_wise"])
def test_spread_embedding_tower_matches_unsharded(kind):
    run_multi_process(_spread_tower_run, world_size=2, kind=kind)


def test_sharded_embedding_tower_matches_unsharded():
    run_multi_process(_tower_run, world_size=2)


def _pool_run(rank, world_size):
    from torchrec_b200.distributed.object_pool import KeyedJaggedTensorPoolSharder, TensorPoolSharder
    from torchrec_b200.distributed.types import ObjectPoolShardingPlan, ObjectPoolShardingType, ShardingEnv
    from torchrec_b200.modules.keyed_jagged_tensor_pool import KeyedJaggedTensorPool
    from torchrec_b200.modules.tensor_pool import TensorPool
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    with MultiProcessContext(rank, world_size, "gloo") as ctx:
        env = ShardingEnv.from_process_group(ctx.pg)
        plan = ObjectPoolShardingPlan(sharding_type=ObjectPoolShardingType.ROW_WISE)
        pool = TensorPoolSharder().shard(TensorPool(pool_size=11, dim=3, dtype=torch.float32), plan, env, torch.device("cpu"))
        assert pool._pool.shape[0] == (4 if rank < 2 else 3)
        ids = torch.tensor([[0, 5, 9], [10, 4, 1], [8, 2, 6]][rank])
        pool.update(ids, ids.float().unsqueeze(1).repeat(1, 3) + 0.5)
        want = torch.tensor([1, 9, 10, 0, 2, 8, 3])  # 3 was never written
        got = pool(want)
        expect = (want.float().unsqueeze(1).repeat(1, 3) + 0.5) * (want != 3).float().unsqueeze(1)
        torch.testing.assert_close(got, expect)
        rep = TensorPoolSharder().shard(TensorPool(pool_size=6, dim=2, dtype=torch.float32), ObjectPoolShardingPlan(sharding_type=ObjectPoolShardingType.REPLICATED_ROW_WISE), env, torch.device("cpu"))
        rep.update(torch.tensor([rank]), torch.full((1, 2), float(rank + 1)))
        torch.testing.assert_close(rep(torch.tensor([0, 1, 2]))[:, 0], torch.tensor([1.0, 2.0, 3.0]))
        kp = KeyedJaggedTensorPoolSharder().shard(KeyedJaggedTensorPool(pool_size=9, feature_max_lengths={"a": 2, "b": 3}), plan, env, torch.device("cpu"))
        my_ids = torch.tensor([[0, 4], [8, 3], [6, 1]][rank])
        kjt = KeyedJaggedTensor(keys=["a", "b"], values=torch.tensor([10, 11, 12, 20, 21, 22, 23]) + 100 * rank, lengths=torch.tensor([2, 1, 1, 3]))
        kp.update(my_ids, kjt)
        out = kp(torch.tensor([3, 0, 7]))  # written by rank 1 (second sample), rank 0 (first sample), never
        assert out.lengths().tolist() == [1, 2, 0, 3, 1, 0]
        assert out["a"].values().tolist() == [112, 10, 11] and out["b"].values().tolist() == [121, 122, 123, 20]


def test_sharded_object_pools():
    run_multi_process(_pool_run, world_size=3)


def _single_embedding_bag(rank, world_size, kind):
    """A plain ``nn.EmbeddingBag`` sharded row-wise / column-wise: forward and one in-backward SGD step against the module itself."""
    import copy

    import torch.distributed as dist

    from torchrec_b200.distributed.embeddingbag import EmbeddingBagSharder, ShardedEmbeddingBag
    from torchrec_b200.distributed.sharding_plan import column_wise, construct_module_sharding_plan, row_wise
    from torchrec_b200.distributed.types import ShardingEnv
    from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward
    from torchrec_b200.test_utils.multi_process import MultiProcessContext

    with MultiProcessContext(rank, world_size, "gloo") as ctx:
        torch.manual_seed(0)
        bag = torch.nn.EmbeddingBag(40, 16, mode="sum", include_last_offset=False)
        local = copy.deepcopy(bag)
        apply_optimizer_in_backward(torch.optim.SGD, local.parameters(), {"lr": 0.1})
        sharder = EmbeddingBagSharder()
        assert sharder.module_type is torch.nn.EmbeddingBag and list(sharder.shardable_parameters(local)) == ["weight"]
        gen = row_wise() if kind == "rw" else column_wise(ranks=[1, 0])
        plan = construct_module_sharding_plan(local, {"weight": gen}, sharder=sharder, world_size=world_size, local_size=world_size, device_type="cpu")
        sharded = sharder.shard(local, plan, ShardingEnv.from_process_group(ctx.pg), torch.device("cpu"))
        assert isinstance(sharded, ShardedEmbeddingBag), type(sharded)
        assert [n for n, _ in sharded.named_parameters()] == ["weight"], [n for n, _ in sharded.named_parameters()]
        sharded.load_state_dict({"weight": _as_sharded_like(sharded.state_dict()["weight"], bag.weight.detach())})
        g = torch.Generator().manual_seed(5)
        inputs, offsets, weights = [], [], []
        for r in range(world_size):
            lens = torch.randint(0, 4, (5,), generator=g)
            inputs.append(torch.randint(0, 40, (int(lens.sum()),), generator=g))
            offsets.append(torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)[:-1]]))
            weights.append(torch.rand(int(lens.sum()), generator=g))
        want_all = [bag(i, o, per_sample_weights=w) for i, o, w in zip(inputs, offsets, weights)]
        got = sharded(inputs[rank], offsets[rank], weights[rank]).wait()
        torch.testing.assert_close(got.detach(), want_all[rank].detach(), rtol=1e-5, atol=1e-6)
        (sum(w.sum() for w in want_all) / world_size).backward()
        got.sum().backward()
        with torch.no_grad():
            want_w = bag.weight - 0.1 * bag.weight.grad
        mine = torch.zeros_like(want_w)
        for s in sharded.state_dict()["weight"].local_shards():
            (r0, c0), (nr, nc) = s.metadata.shard_offsets, s.metadata.shard_sizes
            mine[r0:r0 + nr, c0:c0 + nc] = s.tensor
        dist.all_reduce(mine)
        torch.testing.assert_close(mine, want_w, rtol=1e-5, atol=1e-6)


def _as_sharded_like(template, full):
    """A copy of ``template`` (a ShardedTensor) whose local shards hold the matching blocks of ``full``."""
    import copy

    out = copy.deepcopy(template)
    for s in out.local_shards():
        (r0, c0), (nr, nc) = s.metadata.shard_offsets, s.metadata.shard_sizes
        s.tensor.copy_(full[r0:r0 + nr, c0:c0 + nc])
    return out


@pytest.mark.parametrize("kind", ["rw", "cw"])
def test_single_embedding_bag_sharded(kind):
    run_multi_process(_single_embedding_bag, world_size=2, kind=kind)


def _tower_collection_run(rank, world_size):
    """Two towers in one collection, sharded through the collection sharder: tower 0 on rank 0 (one owner), tower 1 row-wise (spread)."""
    from torchrec_b200.distributed import sharding_plan as sp
    from torchrec_b200.distributed.embedding_tower_sharding import EmbeddingTowerCollectionSharder
    from torchrec_b200.distributed.model_parallel import DistributedModelParallel
    from torchrec_b200.distributed.types import ShardingEnv, ShardingPlan
    from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig
    from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
    from torchrec_b200.modules.embedding_tower import EmbeddingTower, EmbeddingTowerCollection
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    with MultiProcessContext(rank, world_size, "gloo") as ctx:
        torch.manual_seed(0)
        B = 5
        ebc_a = EmbeddingBagCollection(tables=[EmbeddingBagConfig(name="a0", embedding_dim=8, num_embeddings=40, feature_names=["fa"])])
        ebc_b = EmbeddingBagCollection(tables=[EmbeddingBagConfig(name="b0", embedding_dim=8, num_embeddings=60, feature_names=["fb"])])
        g = torch.nn.Module()
        g.towers = EmbeddingTowerCollection([EmbeddingTower(ebc_a, _TowerInteraction(8)), EmbeddingTower(ebc_b, _TowerInteraction(8))])
        l = copy.deepcopy(g)
        sharder = EmbeddingTowerCollectionSharder()
        inner = sharder._tower_sharder._embedding_sharder
        plan = {}
        plan.update(sp.construct_module_sharding_plan(l.towers.towers[0].embedding, {"a0": sp.table_wise(rank=0)}, sharder=inner, world_size=world_size,
                                                      local_size=world_size, device_type="cpu"))
        plan.update(sp.construct_module_sharding_plan(l.towers.towers[1].embedding, {"b0": sp.row_wise()}, sharder=inner, world_size=world_size,
                                                      local_size=world_size, device_type="cpu"))
        dmp = DistributedModelParallel(l, env=ShardingEnv.from_process_group(ctx.pg), device=torch.device("cpu"), plan=ShardingPlan({"towers": plan}),
                                       sharders=sp.get_default_sharders() + [sharder])
        dmp.load_state_dict(copy.deepcopy(g.state_dict()))
        gen = torch.Generator().manual_seed(5)
        per_rank = []
        for r in range(world_size):
            lens = torch.randint(0, 4, (2 * B,), generator=gen)
            vals = torch.cat([torch.randint(0, 40, (int(lens[:B].sum()),), generator=gen), torch.randint(0, 60, (int(lens[B:].sum()),), generator=gen)])
            per_rank.append(KeyedJaggedTensor.from_lengths_sync(keys=["fa", "fb"], values=vals, lengths=lens))
        want = g.towers(per_rank[rank])
        inner_module = dmp.module.module if hasattr(dmp.module, "module") else dmp.module
        got = inner_module.towers(per_rank[rank])
        assert got.shape == (B, 8)
        torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6)
        assert inner_module.towers.towers[0].owner_rank == 0 and inner_module.towers.towers[1].owner_rank == -1


def test_embedding_tower_collection_sharder():
    run_multi_process(_tower_collection_run, world_size=2)
