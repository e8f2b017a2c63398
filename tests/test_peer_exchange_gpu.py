"""Fused sparse engine on real ranks (2 GPUs, NCCL control plane) against the library-collective path: the same sharded
model is built twice, once with ``TRB200_PEER_EXCHANGE=0``; pooled outputs and the tables after three optimizer steps
must agree.  The plan mixes table-wise, row-wise and column-wise tables, one table has two features.

A second test makes one rank arrive late by more than a (shortened) wait limit: the waiting rank's kernels return, its
step raises on the host and nothing faults.  NVLS is off and only plain peer loads / stores are used."""
import copy
import os
import time

import pytest
import torch

from torchrec_b200.test_utils.multi_process import MultiProcessContext, run_multi_process

pytestmark = pytest.mark.gpu

TABLES = [(1000, 128, ["f0"]), (600, 128, ["f1", "f2"]), (33, 128, ["f3"]), (500, 128, ["f4"]), (77, 64, ["f5"])]
KINDS = ["tw", "rw", "tw", "cw", "rw"]


def _make_ebc(pooling):
    from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig
    from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection

    cfgs = [EmbeddingBagConfig(name=f"t{i}", num_embeddings=r, embedding_dim=d, feature_names=list(f), pooling=pooling) for i, (r, d, f) in enumerate(TABLES)]
    return EmbeddingBagCollection(tables=cfgs)


def _make_kjt(B, seed, device):
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    g = torch.Generator().manual_seed(seed)
    keys, lens, vals = [], [], []
    for (r, _, feats) in TABLES:
        for f in feats:
            keys.append(f)
            l = torch.randint(0, 6, (B,), generator=g)
            lens.append(l)
            vals.append(torch.randint(0, r, (int(l.sum()),), generator=g))
    return KeyedJaggedTensor.from_lengths_sync(keys=keys, values=torch.cat(vals), lengths=torch.cat(lens)).to(device)


class _Model(torch.nn.Module):
    def __init__(self, ebc):
        super().__init__()
        self.ebc = ebc
        self.over = torch.nn.Linear(sum(len(f) * d for _, d, f in TABLES), 1)

    def forward(self, kjt):
        kt = self.ebc(kjt)
        v = kt.values().float()
        return self.over(v), v


def _build(ctx, world_size, pooling, peer):
    from torchrec_b200.distributed import sharding_plan as sp
    from torchrec_b200.distributed.embeddingbag import EmbeddingBagCollectionSharder
    from torchrec_b200.distributed.model_parallel import DistributedModelParallel
    from torchrec_b200.distributed.types import ShardingEnv, ShardingPlan
    from torchrec_b200.modules.embedding_configs import DataType
    from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward
    from torchrec_b200.optim.rowwise_adagrad import RowWiseAdagrad

    os.environ["TRB200_PEER_EXCHANGE"] = "1" if peer else "0"
    torch.manual_seed(0)
    model = _Model(_make_ebc(pooling))
    apply_optimizer_in_backward(RowWiseAdagrad, model.ebc.parameters(), {"lr": 0.1, "eps": 1e-8})
    sharder = EmbeddingBagCollectionSharder(fused_params={"output_dtype": DataType.BF16})
    gens = {}
    for i, kind in enumerate(KINDS):
        gens[f"t{i}"] = {"tw": sp.table_wise(rank=[1, 0, 1, 1, 0][i]), "rw": sp.row_wise(), "cw": sp.column_wise(ranks=[1, 0])}[kind]
    plan = ShardingPlan({"ebc": sp.construct_module_sharding_plan(model.ebc, gens, sharder=sharder, world_size=world_size, local_size=world_size, device_type="cuda")})
    return DistributedModelParallel(model, env=ShardingEnv.from_process_group(ctx.pg), device=ctx.device, plan=plan, sharders=[sharder])


def _sharded_ebc(dmp):
    from torchrec_b200.distributed.embeddingbag import ShardedEmbeddingBagCollection

    return [m for m in dmp.modules() if isinstance(m, ShardedEmbeddingBagCollection)][0]


def _run(rank, world_size, pooling_name):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from torchrec_b200.distributed.peer_memory import check_all
    from torchrec_b200.modules.embedding_configs import PoolingType

    with MultiProcessContext(rank, world_size, "nccl") as ctx:
        pooling = PoolingType[pooling_name]
        ref = _build(ctx, world_size, pooling, peer=False)
        fused = _build(ctx, world_size, pooling, peer=True)
        fused.load_state_dict(copy.deepcopy(ref.state_dict()))
        opt_r = torch.optim.SGD([p for n, p in ref.named_parameters() if "ebc" not in n], lr=0.05)
        opt_f = torch.optim.SGD([p for n, p in fused.named_parameters() if "ebc" not in n], lr=0.05)
        B = 300
        for step in range(3):
            kjt = _make_kjt(B, 100 + 10 * step + rank, ctx.device)
            opt_r.zero_grad(); opt_f.zero_grad()
            os.environ["TRB200_PEER_EXCHANGE"] = "0"
            pr, vr = ref(kjt)
            os.environ["TRB200_PEER_EXCHANGE"] = "1"
            pf, vf = fused(kjt)
            torch.testing.assert_close(vf, vr, rtol=2e-2, atol=2e-2)  # bf16 outputs on both paths (fp16 wire on the reference one)
            pr.mean().backward()
            pf.mean().backward()
            opt_r.step(); opt_f.step()
        torch.cuda.synchronize()
        check_all()
        assert _sharded_ebc(fused)._engine is not None, "the fused sparse engine must be active on a 2-GPU node"
        assert _sharded_ebc(ref)._engine is None
        sd_r, sd_f = ref.state_dict(), fused.state_dict()
        for name, vr in sd_r.items():
            vf = sd_f[name]
            if hasattr(vr, "local_shards"):
                for a, b in zip(vf.local_shards(), vr.local_shards()):
                    torch.testing.assert_close(a.tensor, b.tensor, rtol=2e-2, atol=2e-3)
            else:
                torch.testing.assert_close(vf, vr, rtol=2e-2, atol=2e-3)


@pytest.mark.parametrize("pooling_name", ["SUM", "MEAN"])
def test_engine_matches_library_collectives(pooling_name):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    run_multi_process(_run, world_size=2, pooling_name=pooling_name)


def _run_late(rank, world_size):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["TRB200_PEER_WAIT_S"] = "0.5"
    from torchrec_b200.distributed.peer_memory import check_all
    from torchrec_b200.modules.embedding_configs import PoolingType

    with MultiProcessContext(rank, world_size, "nccl") as ctx:
        model = _build(ctx, world_size, PoolingType.SUM, peer=True)
        kjt = _make_kjt(64, rank, ctx.device)
        model(kjt)  # sizes the buffers, both ranks in step
        torch.cuda.synchronize()
        check_all()
        import torch.distributed as dist

        dist.barrier(group=ctx.pg)
        if rank == 1:
            time.sleep(3.0)  # far past the 0.5 s wait limit: rank 0's kernels give up and return
        _, v = model(kjt)
        torch.cuda.synchronize()
        if rank == 0:
            assert torch.isnan(v).any(), "a step whose wait ran out must not hand on stale rows"
            with pytest.raises(RuntimeError, match="timed out waiting for rank 1"):
                check_all()
        dist.barrier(group=ctx.pg)


def test_late_rank_raises_on_the_waiting_rank():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    run_multi_process(_run_late, world_size=2)
