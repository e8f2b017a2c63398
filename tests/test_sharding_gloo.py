"""Sharded-vs-unsharded parity on CPU/gloo, world size 2: one optimizer step on a global model and on
its sharded copy must give the same predictions and the same updated tables (cf. the reference's
``torchrec/distributed/test_utils/test_sharding.py:760-1037``)."""
import copy

import pytest
import torch
import torch.distributed as dist

from torchrec_b200.test_utils.multi_process import MultiProcessContext, run_multi_process

TABLES = [(100, 16, ["f0"]), (60, 16, ["f1", "f2"]), (33, 16, ["f3"]), (50, 16, ["f4"])]


def _make_ebc(pooling, weighted=False):
    from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig, PoolingType
    from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection

    cfgs = [EmbeddingBagConfig(name=f"t{i}", num_embeddings=r, embedding_dim=d, feature_names=list(f), pooling=pooling) for i, (r, d, f) in enumerate(TABLES)]
    return EmbeddingBagCollection(tables=cfgs, is_weighted=weighted)


def _make_kjt(B, seed, weighted=False):
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    g = torch.Generator().manual_seed(seed)
    keys, lens, vals = [], [], []
    for (r, _, feats) in TABLES:
        for f in feats:
            keys.append(f)
            l = torch.randint(0, 5, (B,), generator=g)
            lens.append(l)
            vals.append(torch.randint(0, r, (int(l.sum()),), generator=g))
    values = torch.cat(vals)
    w = torch.rand(values.numel(), generator=g) if weighted else None
    # shuffle key order relative to table order to exercise the feature permute
    order = [4, 0, 3, 1, 2]
    kjt = KeyedJaggedTensor.from_lengths_sync(keys=keys, values=values, lengths=torch.cat(lens), weights=w)
    return kjt.permute(order)


def _plan_for(ebc, sharding, world_size, rank_fn=None):
    from torchrec_b200.distributed import sharding_plan as sp
    from torchrec_b200.distributed.embeddingbag import EmbeddingBagCollectionSharder

    gens = {}
    for i, cfg in enumerate(ebc.embedding_bag_configs()):
        if sharding == "tw":
            gens[cfg.name] = sp.table_wise(rank=i % world_size)
        elif sharding == "rw":
            gens[cfg.name] = sp.row_wise()
        elif sharding == "cw":
            gens[cfg.name] = sp.column_wise(ranks=[(i + j) % world_size for j in range(2)])
        elif sharding == "dp":
            gens[cfg.name] = sp.data_parallel()
        elif sharding == "twrw":
            gens[cfg.name] = sp.table_row_wise(host_index=0)
        elif sharding == "grid":
            gens[cfg.name] = sp.grid_shard(host_indexes=[0, 0] if world_size == 2 else [0, 1])
        elif sharding == "mixed":
            gens[cfg.name] = [sp.table_wise(rank=0), sp.row_wise(), sp.column_wise(ranks=[1, 0]), sp.table_wise(rank=1)][i]
        elif sharding == "mixed_nocw":
            # row-wise optimizer state of a column shard is computed from the shard's own columns, so
            # column-wise tables do not reproduce the unsharded row-wise Adagrad step exactly
            gens[cfg.name] = [sp.table_wise(rank=0), sp.row_wise(), sp.row_wise(), sp.table_wise(rank=1)][i]
    return sp.construct_module_sharding_plan(ebc, gens, sharder=EmbeddingBagCollectionSharder(), world_size=world_size, local_size=world_size, device_type="cpu")


class _Model(torch.nn.Module):
    def __init__(self, ebc):
        super().__init__()
        self.ebc = ebc
        n = sum(len(f) for _, _, f in TABLES) * 16
        self.over = torch.nn.Linear(n, 1)

    def forward(self, kjt):
        kt = self.ebc(kjt)
        return self.over(kt.values() if hasattr(kt, "values") else kt), kt


def _parity(rank, world_size, sharding, pooling_name, opt_name, weighted=False, tables=None):
    if tables is not None:
        global TABLES
        TABLES = tables
    from torchrec_b200.distributed.model_parallel import DistributedModelParallel
    from torchrec_b200.distributed.types import ShardingEnv, ShardingPlan
    from torchrec_b200.modules.embedding_configs import PoolingType
    from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward
    from torchrec_b200.optim.rowwise_adagrad import RowWiseAdagrad

    pooling = PoolingType[pooling_name]
    with MultiProcessContext(rank, world_size, "gloo") as ctx:
        torch.manual_seed(0)
        B = 6
        global_model = _Model(_make_ebc(pooling, weighted))
        local_model = copy.deepcopy(global_model)
        lr = 0.1
        if opt_name == "rowwise_adagrad":
            opt_cls, kw = RowWiseAdagrad, {"lr": lr, "eps": 1e-8}
        else:
            opt_cls, kw = torch.optim.SGD, {"lr": lr}
        if sharding != "dp":
            apply_optimizer_in_backward(opt_cls, local_model.ebc.parameters(), kw)
        plan = ShardingPlan({"ebc": _plan_for(local_model.ebc, sharding, world_size)})
        dmp = DistributedModelParallel(local_model, env=ShardingEnv.from_process_group(ctx.pg), device=torch.device("cpu"), plan=plan)
        # same weights everywhere: load the global state dict into the sharded model
        dmp.load_state_dict(copy.deepcopy(global_model.state_dict()))
        dense_params = [p for n, p in dmp.named_parameters() if "ebc" not in n or sharding == "dp"]
        dense_opt = torch.optim.SGD(dense_params, lr=lr)
        g_emb_opt = opt_cls(global_model.ebc.parameters(), **kw) if sharding != "dp" else torch.optim.SGD(global_model.ebc.parameters(), lr=lr)
        g_dense_opt = torch.optim.SGD(global_model.over.parameters(), lr=lr)

        kjts = [_make_kjt(B, 100 + r, weighted) for r in range(world_size)]
        # global batch = concatenation of the per-rank batches
        from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor
        keys = kjts[0].keys()
        vals, lens, ws = [], [], []
        for k in keys:
            for kj in kjts:
                jt = kj[k]
                vals.append(jt.values()); lens.append(jt.lengths())
                if weighted:
                    ws.append(jt.weights())
        global_kjt = KeyedJaggedTensor.from_lengths_sync(keys=keys, values=torch.cat(vals), lengths=torch.cat(lens), weights=torch.cat(ws) if weighted else None)

        for step in range(2):
            # ---- global
            g_emb_opt.zero_grad(); g_dense_opt.zero_grad()
            g_pred, g_kt = global_model(global_kjt)
            g_loss = g_pred.view(world_size, B).mean()  # mean over ranks of per-rank sums / B ... use mean
            g_loss = g_pred.mean()
            g_loss.backward()
            g_emb_opt.step(); g_dense_opt.step()
            # ---- local
            dense_opt.zero_grad()
            l_pred, l_kt = dmp(kjts[rank])
            l_loss = l_pred.mean()
            l_loss.backward()
            dense_opt.step()
            torch.testing.assert_close(l_pred.detach(), g_pred.detach().view(world_size, B, 1)[rank] if False else g_pred.detach()[_rows(keys, rank, B, world_size)], rtol=1e-4, atol=1e-5)

        # tables after two steps: gather the sharded state dict and compare with the global model
        sd = dmp.state_dict()
        for name, gt in global_model.state_dict().items():
            v = sd[name]
            if hasattr(v, "local_shards"):
                full = torch.zeros_like(gt)
                mine = torch.zeros_like(gt)
                for s in v.local_shards():
                    ro, co = s.metadata.shard_offsets
                    rs, cs = s.metadata.shard_sizes
                    mine[ro:ro + rs, co:co + cs] = s.tensor
                dist.all_reduce(mine)
                full = mine
                torch.testing.assert_close(full, gt, rtol=1e-4, atol=1e-5)
            else:
                torch.testing.assert_close(v, gt, rtol=1e-4, atol=1e-5)


def _rows(keys, rank, B, W):
    return slice(rank * B, (rank + 1) * B)


@pytest.mark.parametrize("sharding", ["tw", "rw", "cw", "dp", "twrw", "grid", "mixed"])
def test_sharding_parity_sum_sgd(sharding):
    run_multi_process(_parity, world_size=2, sharding=sharding, pooling_name="SUM", opt_name="sgd")


@pytest.mark.parametrize("sharding", ["tw", "rw", "mixed_nocw"])
def test_sharding_parity_mean_rowwise_adagrad(sharding):
    run_multi_process(_parity, world_size=2, sharding=sharding, pooling_name="MEAN", opt_name="rowwise_adagrad")


def test_sharding_parity_weighted():
    run_multi_process(_parity, world_size=2, sharding="mixed", pooling_name="SUM", opt_name="sgd", weighted=True)


def test_sharding_rw_more_ranks_than_rows():
    """Row-wise tables with fewer rows than ranks leave some ranks with empty shards (weights and row-wise state)."""
    tables = [(3, 16, ["f0"]), (60, 16, ["f1", "f2"]), (2, 16, ["f3"]), (50, 16, ["f4"])]
    run_multi_process(_parity, world_size=4, sharding="rw", pooling_name="SUM", opt_name="rowwise_adagrad", tables=tables)
