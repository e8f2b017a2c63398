"""State dicts with DTensor / ShardedTensor shards and a ``torch.distributed.checkpoint`` round trip across plans:
saved under plan A (column-wise, two shards per rank for one table), loaded under plan B (row-wise), gloo world of 2."""
import os
import shutil
import tempfile

import torch

from torchrec_b200.test_utils.multi_process import MultiProcessContext, run_multi_process

TABLES = [(40, 16, ["f0"]), (24, 32, ["f1"])]


def _build(ctx, kinds, output_dtensor):
    from torchrec_b200.distributed import sharding_plan as sp
    from torchrec_b200.distributed.embeddingbag import EmbeddingBagCollectionSharder
    from torchrec_b200.distributed.model_parallel import DistributedModelParallel
    from torchrec_b200.distributed.types import ShardingEnv, ShardingPlan
    from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig
    from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
    from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward
    from torchrec_b200.optim.rowwise_adagrad import RowWiseAdagrad

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.ebc = EmbeddingBagCollection([EmbeddingBagConfig(name=f"t{i}", num_embeddings=r, embedding_dim=d, feature_names=f) for i, (r, d, f) in enumerate(TABLES)])

        def forward(self, kjt):
            return self.ebc(kjt).values()

    m = M()
    apply_optimizer_in_backward(RowWiseAdagrad, m.ebc.parameters(), {"lr": 0.1})
    sharder = EmbeddingBagCollectionSharder()
    gens = {}
    for i, k in enumerate(kinds):
        gens[f"t{i}"] = {"cw2": sp.column_wise(ranks=[0, 1, 0, 1]) if TABLES[i][1] >= 32 else sp.column_wise(ranks=[0, 1]), "rw": sp.row_wise(), "tw": sp.table_wise(rank=i % 2)}[k]
    plan = ShardingPlan({"ebc": sp.construct_module_sharding_plan(m.ebc, gens, sharder=sharder, world_size=2, local_size=2, device_type="cpu")})
    env = ShardingEnv.from_process_group(ctx.pg)
    env.output_dtensor = output_dtensor
    return DistributedModelParallel(m, env=env, device=torch.device("cpu"), plan=plan, sharders=[sharder])


def _full_table(dmp, name, rows, cols):
    """Reassemble a table from the shards of every rank."""
    import torch.distributed as dist

    v = dmp.state_dict()[name]
    if type(v).__name__ == "DTensor":
        inner = v.to_local()
        mine = [(tuple(int(x) for x in o), s.clone()) for s, o in zip(inner.local_shards(), inner.local_offsets())]
    else:
        mine = [(tuple(sh.metadata.shard_offsets), sh.tensor.clone()) for sh in v.local_shards()]
    everyone = [None, None]
    dist.all_gather_object(everyone, mine)
    full = torch.zeros(rows, cols)
    for pieces in everyone:
        for (ro, co), t in pieces:
            full[ro: ro + t.shape[0], co: co + t.shape[1]] = t
    return full


def _run(rank, world_size, dtensor, tmp):
    import torch.distributed.checkpoint as dcp

    with MultiProcessContext(rank, world_size, "gloo") as ctx:
        a = _build(ctx, ["rw", "cw2"], dtensor)
        sd_a = a.state_dict()
        v = sd_a["ebc.embedding_bags.t1.weight"]
        if dtensor:
            assert type(v).__name__ == "DTensor" and len(v.to_local().local_shards()) == 2 and tuple(v.shape) == (24, 32)
            assert type(sd_a["ebc.embedding_bags.t0.weight"]).__name__ == "DTensor"
        else:
            assert hasattr(v, "local_shards") and len(v.local_shards()) == 2
        # the in-backward optimizer's states leave in the same form as the tables
        opt_state = a.fused_optimizer.state_dict()["state"]
        sharded_states = [v for per_param in opt_state.values() for v in per_param.values() if not isinstance(v, (int, float)) and type(v).__name__ in ("DTensor", "ShardedTensor")]
        assert sharded_states, "the row-wise Adagrad state of sharded tables is missing"
        assert all(type(v).__name__ == ("DTensor" if dtensor else "ShardedTensor") for v in sharded_states), [type(v).__name__ for v in sharded_states]
        if dtensor:
            rowwise = [v for v in sharded_states if len(v.shape) == 1]
            assert rowwise and all(sum(int(s.shape[0]) for s in v.to_local().local_shards()) > 0 for v in rowwise)
        want = {f"ebc.embedding_bags.t{i}.weight": _full_table(a, f"ebc.embedding_bags.t{i}.weight", r, d) for i, (r, d, _) in enumerate(TABLES)}
        dcp.save(sd_a, checkpoint_id=tmp)
        b = _build(ctx, ["cw2" if False else "tw", "rw"], dtensor)  # another layout: table-wise and row-wise
        sd_b = b.state_dict()
        dcp.load(sd_b, checkpoint_id=tmp)
        b.load_state_dict(sd_b)
        for i, (r, d, _) in enumerate(TABLES):
            key = f"ebc.embedding_bags.t{i}.weight"
            torch.testing.assert_close(_full_table(b, key, r, d), want[key])


def _roundtrip(dtensor):
    tmp = tempfile.mkdtemp(prefix="trb_dcp_")
    try:
        run_multi_process(_run, world_size=2, dtensor=dtensor, tmp=tmp)
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


def test_dcp_roundtrip_sharded_tensor():
    _roundtrip(False)


def test_dcp_roundtrip_dtensor():
    _roundtrip(True)
