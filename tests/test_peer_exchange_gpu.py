"""Fused lookup + exchange over peer-mapped buffers (2 GPUs) against the library all-to-all path: the same sharded
model is built twice, once with ``TRB200_PEER_EXCHANGE=0``; pooled outputs and the tables after two optimizer steps
must agree.  Also checks the device-side barrier's bounded wait path on the host side of its API."""
import copy
import os

import pytest
import torch

from torchrec_b200.test_utils.multi_process import MultiProcessContext, run_multi_process

pytestmark = pytest.mark.gpu

TABLES = [(1000, 128, ["f0"]), (600, 128, ["f1", "f2"]), (33, 128, ["f3"]), (500, 128, ["f4"]), (77, 128, ["f5"])]


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
        self.over = torch.nn.Linear(sum(len(f) for _, _, f in TABLES) * 128, 1)

    def forward(self, kjt):
        kt = self.ebc(kjt)
        v = kt.values().float()
        return self.over(v), v


def _build(ctx, rank, world_size, pooling, peer):
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
    # ranks [1, 0, 1, 1, 0]: rank 0 owns two tables, rank 1 three; t1 has two features
    gens = {f"t{i}": sp.table_wise(rank=[1, 0, 1, 1, 0][i]) for i in range(len(TABLES))}
    plan = ShardingPlan({"ebc": sp.construct_module_sharding_plan(model.ebc, gens, sharder=sharder, world_size=world_size, local_size=world_size, device_type="cuda")})
    return DistributedModelParallel(model, env=ShardingEnv.from_process_group(ctx.pg), device=ctx.device, plan=plan, sharders=[sharder])


def _run(rank, world_size, pooling_name):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from torchrec_b200.distributed.embedding_lookup import GroupedPooledEmbeddingsLookup
    from torchrec_b200.modules.embedding_configs import PoolingType

    with MultiProcessContext(rank, world_size, "nccl") as ctx:
        pooling = PoolingType[pooling_name]
        ref = _build(ctx, rank, world_size, pooling, peer=False)
        fused = _build(ctx, rank, world_size, pooling, peer=True)
        fused.load_state_dict(copy.deepcopy(ref.state_dict()))
        def lookups_of(dmp):
            from torchrec_b200.distributed.embeddingbag import ShardedEmbeddingBagCollection

            out = []
            for m in dmp.modules():
                if isinstance(m, ShardedEmbeddingBagCollection):
                    out += [l for l in m._lookups if isinstance(l, GroupedPooledEmbeddingsLookup)]
            return out

        lookups = lookups_of(fused)
        assert lookups and all(m._peer is not None for m in lookups), "the fused exchange must be active on a 2-GPU node"
        assert all(m._peer is None for m in lookups_of(ref))
        opt_r = torch.optim.SGD([p for n, p in ref.named_parameters() if "ebc" not in n], lr=0.05)
        opt_f = torch.optim.SGD([p for n, p in fused.named_parameters() if "ebc" not in n], lr=0.05)
        B = 64
        for step in range(3):
            kjt = _make_kjt(B, 100 + 10 * step + rank, ctx.device)
            opt_r.zero_grad(); opt_f.zero_grad()
            pr, vr = ref(kjt)
            pf, vf = fused(kjt)
            torch.testing.assert_close(vf, vr, rtol=2e-2, atol=2e-2)  # bf16 outputs on both paths (fp16 wire on the reference one)
            pr.mean().backward()
            pf.mean().backward()
            opt_r.step(); opt_f.step()
        torch.cuda.synchronize()
        for m in lookups:
            m._peer.check_error()
        # the tables were placed out of order, so the exchange stored them at their final columns instead of permuting afterwards
        assert all(m._peer_feature_columns is not None for m in lookups)
        sd_r, sd_f = ref.state_dict(), fused.state_dict()
        for name, vr in sd_r.items():
            vf = sd_f[name]
            if hasattr(vr, "local_shards"):
                for a, b in zip(vf.local_shards(), vr.local_shards()):
                    torch.testing.assert_close(a.tensor, b.tensor, rtol=2e-2, atol=2e-3)
            else:
                torch.testing.assert_close(vf, vr, rtol=2e-2, atol=2e-3)


@pytest.mark.parametrize("pooling_name", ["SUM", "MEAN"])
def test_peer_exchange_matches_all_to_all(pooling_name):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    run_multi_process(_run, world_size=2, pooling_name=pooling_name)
