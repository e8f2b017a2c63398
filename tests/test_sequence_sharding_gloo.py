"""Sharded ``EmbeddingCollection`` against the unsharded module on CPU/gloo, world size 2: per-feature
jagged outputs and the tables after two optimizer steps must agree (cf. the reference's
``torchrec/distributed/tests/test_sequence_model_parallel.py``)."""
import copy

import pytest
import torch
import torch.distributed as dist

from torchrec_b200.test_utils.multi_process import MultiProcessContext, run_multi_process

TABLES = [(100, 16, ["f0"]), (60, 16, ["f1", "f2"]), (33, 16, ["f3"])]
KEY_ORDER = [3, 0, 2, 1]


def _make_ec():
    from torchrec_b200.modules.embedding_configs import EmbeddingConfig
    from torchrec_b200.modules.embedding_modules import EmbeddingCollection

    cfgs = [EmbeddingConfig(name=f"t{i}", num_embeddings=r, embedding_dim=d, feature_names=list(f)) for i, (r, d, f) in enumerate(TABLES)]
    return EmbeddingCollection(tables=cfgs)


def _make_kjt(B, seed, dup=False):
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    g = torch.Generator().manual_seed(seed)
    keys, lens, vals = [], [], []
    for (r, _, feats) in TABLES:
        for f in feats:
            keys.append(f)
            l = torch.randint(0, 5, (B,), generator=g)
            lens.append(l)
            vals.append(torch.randint(0, 6 if dup else r, (int(l.sum()),), generator=g))
    kjt = KeyedJaggedTensor.from_lengths_sync(keys=keys, values=torch.cat(vals), lengths=torch.cat(lens))
    return kjt.permute(KEY_ORDER)


def _plan_for(ec, sharding, world_size):
    from torchrec_b200.distributed import sharding_plan as sp
    from torchrec_b200.distributed.embedding import EmbeddingCollectionSharder

    gens = {}
    for i, cfg in enumerate(ec.embedding_configs()):
        if sharding == "tw":
            gens[cfg.name] = sp.table_wise(rank=i % world_size)
        elif sharding == "rw":
            gens[cfg.name] = sp.row_wise()
        elif sharding == "cw":
            gens[cfg.name] = sp.column_wise(ranks=[(i + 1 + j) % world_size for j in range(2)])
        elif sharding == "dp":
            gens[cfg.name] = sp.data_parallel()
        elif sharding == "mixed":
            gens[cfg.name] = [sp.table_wise(rank=1), sp.row_wise(), sp.column_wise(ranks=[1, 0])][i]
    return sp.construct_module_sharding_plan(ec, gens, sharder=EmbeddingCollectionSharder(), world_size=world_size, local_size=world_size, device_type="cpu")


class _Model(torch.nn.Module):
    def __init__(self, ec):
        super().__init__()
        self.ec = ec
        self.proj = torch.nn.Linear(16, 1)

    def forward(self, kjt):
        jts = self.ec(kjt)
        if hasattr(jts, "wait"):
            jts = jts.wait()
        loss = sum(self.proj(jt.values()).sum() * (i + 1) for i, (_, jt) in enumerate(sorted(jts.items())))
        return loss, jts


def _parity(rank, world_size, sharding, dedup=False):
    from torchrec_b200.distributed.embedding import EmbeddingCollectionSharder
    from torchrec_b200.distributed.model_parallel import DistributedModelParallel
    from torchrec_b200.distributed.types import ShardingEnv, ShardingPlan
    from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    with MultiProcessContext(rank, world_size, "gloo") as ctx:
        torch.manual_seed(0)
        B = 5
        global_model = _Model(_make_ec())
        local_model = copy.deepcopy(global_model)
        lr = 0.1
        if sharding != "dp":
            apply_optimizer_in_backward(torch.optim.SGD, local_model.ec.parameters(), {"lr": lr})
        plan = ShardingPlan({"ec": _plan_for(local_model.ec, sharding, world_size)})
        dmp = DistributedModelParallel(
            local_model, env=ShardingEnv.from_process_group(ctx.pg), device=torch.device("cpu"), plan=plan,
            sharders=[EmbeddingCollectionSharder(use_index_dedup=dedup)],
        )
        dmp.load_state_dict(copy.deepcopy(global_model.state_dict()))
        dense_params = [p for n, p in dmp.named_parameters() if "ec." not in n or sharding == "dp"]
        dense_opt = torch.optim.SGD(dense_params, lr=lr)
        g_opt = torch.optim.SGD(global_model.parameters(), lr=lr)
        kjts = [_make_kjt(B, 100 + r, dup=dedup) for r in range(world_size)]
        for step in range(2):
            # the global model sees every rank's batch in turn and sums the losses: same gradient as the
            # sharded model whose dense part is all-reduced with SUM semantics emulated below
            g_opt.zero_grad()
            g_losses, g_outs = [], []
            for r in range(world_size):
                l, o = global_model(kjts[r])
                g_losses.append(l)
                g_outs.append(o)
            (sum(g_losses) / world_size).backward()
            # (the sequence all-to-all divides gradients by the world size, DDP averages: both match the mean loss)
            dense_opt.zero_grad()
            l_loss, l_out = dmp(kjts[rank])
            for k, jt in g_outs[rank].items():
                torch.testing.assert_close(l_out[k].values().detach(), jt.values().detach(), rtol=1e-5, atol=1e-6)
                assert torch.equal(l_out[k].lengths(), jt.lengths())
            l_loss.backward()
            dense_opt.step()
            g_opt.step()
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
                torch.testing.assert_close(mine, gt, rtol=1e-4, atol=1e-5)
            else:
                torch.testing.assert_close(v, gt, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("sharding", ["tw", "rw", "cw", "dp", "mixed"])
def test_sequence_sharding_parity(sharding):
    run_multi_process(_parity, world_size=2, sharding=sharding)


@pytest.mark.parametrize("sharding", ["tw", "rw"])
def test_sequence_sharding_index_dedup(sharding):
    run_multi_process(_parity, world_size=2, sharding=sharding, dedup=True)


def _write_rows(rank, world_size):
    """Online row writes: every rank writes a few rows; afterwards the assembled tables hold them, whatever the sharding."""
    from torchrec_b200.distributed.embedding import EmbeddingCollectionSharder
    from torchrec_b200.distributed.model_parallel import DistributedModelParallel
    from torchrec_b200.distributed.types import ShardingEnv, ShardingPlan
    from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    with MultiProcessContext(rank, world_size, "gloo") as ctx:
        torch.manual_seed(0)
        reference = _Model(_make_ec())
        local_model = copy.deepcopy(reference)
        apply_optimizer_in_backward(torch.optim.SGD, local_model.ec.parameters(), {"lr": 0.1})
        plan = ShardingPlan({"ec": _plan_for(local_model.ec, "mixed", world_size)})  # t0 table-wise, t1 row-wise, t2 column-wise
        dmp = DistributedModelParallel(local_model, env=ShardingEnv.from_process_group(ctx.pg), device=torch.device("cpu"), plan=plan,
                                       sharders=[EmbeddingCollectionSharder()])
        dmp.load_state_dict(copy.deepcopy(reference.state_dict()))
        # rank r writes rows 10+r and 50+r of t1 (through f2), row 3+r of t0 and row 20+r of t2
        ids = {"f0": [3 + rank], "f2": [10 + rank, 50 + rank], "f3": [20 + rank]}
        keys = list(ids)
        values = torch.tensor([i for k in keys for i in ids[k]])
        rows = torch.arange(values.numel() * 16, dtype=torch.float32).view(-1, 16) + 1000 * (rank + 1)
        kjt = KeyedJaggedTensor(keys=keys, values=values, weights=rows, lengths=torch.tensor([len(ids[k]) for k in keys]), stride=1)
        sharded_ec = dmp.module.ec
        sharded_ec.write(kjt)
        want = {n: t.clone() for n, t in reference.state_dict().items()}
        for r in range(world_size):
            r_rows = torch.arange(4 * 16, dtype=torch.float32).view(-1, 16) + 1000 * (r + 1)
            want["ec.embeddings.t0.weight"][3 + r] = r_rows[0]
            want["ec.embeddings.t1.weight"][10 + r] = r_rows[1]
            want["ec.embeddings.t1.weight"][50 + r] = r_rows[2]
            want["ec.embeddings.t2.weight"][20 + r] = r_rows[3]
        sd = dmp.state_dict()
        for name in ("ec.embeddings.t0.weight", "ec.embeddings.t1.weight", "ec.embeddings.t2.weight"):
            mine = torch.zeros_like(want[name])
            for s in sd[name].local_shards():
                ro, co = s.metadata.shard_offsets
                rs, cs = s.metadata.shard_sizes
                mine[ro:ro + rs, co:co + cs] = s.tensor
            dist.all_reduce(mine)
            torch.testing.assert_close(mine, want[name], rtol=0, atol=0)


def test_embedding_rows_can_be_written_online():
    run_multi_process(_write_rows, world_size=2)
