"""Fused sparse engine on real ranks (2 GPUs, NCCL control plane) against the unsharded tables in plain fp32 torch: pooled
outputs of every step and the tables after three optimizer steps (row-wise Adagrad written out in torch over the global
batch) must agree.  The plan mixes table-wise, row-wise and column-wise tables, one table has two features.

A second test makes one rank arrive late by more than a (shortened) wait limit: the waiting rank's kernels return, its
step raises on the host and nothing faults.  NVLS is off and only plain peer loads / stores are used."""
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


def _oracle_forward(full, kjt, B, mean):
    """Pooled output of the unsharded tables in plain fp32 torch."""
    off = kjt.offsets().long().cpu()
    vals = kjt.values().long()
    outs, k = [], 0
    for ti, (_, d, feats) in enumerate(TABLES):
        for _ in feats:
            s, e = int(off[k * B]), int(off[(k + 1) * B])
            o = (off[k * B:(k + 1) * B] - s).to(vals.device)
            res = torch.nn.functional.embedding_bag(vals[s:e], full[ti], o, mode="sum") if e > s else torch.zeros(B, d, device=vals.device)
            if mean:
                res = res / (off[k * B + 1:(k + 1) * B + 1] - off[k * B:(k + 1) * B]).clamp(min=1).to(vals.device).float().unsqueeze(1)
            outs.append(res)
            k += 1
    return torch.cat(outs, dim=1)


def _oracle_update(full, state, kjts, B, mean, grad_row, lr, eps, world):
    """Row-wise Adagrad on the unsharded tables for the global batch: every bag of every rank contributes ``grad_row`` (the
    same output gradient for all samples of this test's loss) to its rows; column-wise shards keep one state per column block."""
    col, k = 0, 0
    for ti, (rows, d, feats) in enumerate(TABLES):
        gsum = torch.zeros(rows, d, device=full[ti].device)
        for fi in range(len(feats)):
            g = grad_row[col: col + d]
            for kjt in kjts:
                off = kjt.offsets().long()
                vals = kjt.values().long()
                s, e = int(off[k * B]), int(off[(k + 1) * B])
                lens = off[k * B + 1:(k + 1) * B + 1] - off[k * B:(k + 1) * B]
                w = torch.repeat_interleave(1.0 / lens.clamp(min=1).float() if mean else torch.ones_like(lens, dtype=torch.float32), lens)
                gsum.index_add_(0, vals[s:e], w.unsqueeze(1) * g.unsqueeze(0))
            col += d
            k += 1
        blocks = [(0, d)] if KINDS[ti] != "cw" else [(0, d // 2), (d // 2, d)]
        touched = torch.zeros(rows, dtype=torch.bool, device=gsum.device)
        for kjt in kjts:
            pass
        touched = gsum.abs().sum(1) > 0
        for bi, (c0, c1) in enumerate(blocks):
            gb = gsum[:, c0:c1]
            state[ti][bi] += torch.where(touched, gb.pow(2).mean(1), torch.zeros_like(gb[:, 0]))
            upd = lr * gb / (state[ti][bi].sqrt() + eps).unsqueeze(1)
            full[ti][:, c0:c1] -= torch.where(touched.unsqueeze(1), upd, torch.zeros_like(upd))


def _run(rank, world_size, pooling_name):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["TRB200_PEER_WAIT_S"] = "5"  # a protocol error shows up as a named time-out, not as a long stall
    import faulthandler

    import torch.distributed as dist

    faulthandler.dump_traceback_later(100, exit=True)
    from torchrec_b200.distributed.peer_memory import check_all
    from torchrec_b200.modules.embedding_configs import PoolingType

    with MultiProcessContext(rank, world_size, "nccl") as ctx:
        mean = pooling_name == "MEAN"
        fused = _build(ctx, world_size, PoolingType[pooling_name], peer=True)
        # known weights: the unsharded tables, loaded through the state dict (full-size tensors are cut into the local shards)
        g = torch.Generator().manual_seed(5)
        full = [(torch.randn(r, d, generator=g) * 0.1).to(ctx.device) for r, d, _ in TABLES]
        sd = dict(fused.state_dict())
        for i in range(len(TABLES)):
            sd[f"ebc.embedding_bags.t{i}.weight"] = full[i].clone()
        fused.load_state_dict(sd)
        state = [[torch.zeros(r, device=ctx.device) for _ in range(2)] for r, _, _ in TABLES]
        B = 300
        for step in range(3):
            kjt = _make_kjt(B, 100 + 10 * step + rank, ctx.device)
            pf, vf = fused(kjt)
            want = _oracle_forward(full, kjt, B, mean)
            torch.testing.assert_close(vf, want, rtol=2e-2, atol=2e-2)  # bf16 output, fp16 staging
            over_w = [m for m in fused.modules() if isinstance(m, torch.nn.Linear)][0].weight.detach().clone()
            pf.mean().backward()
            gathered = [None] * world_size
            dist.all_gather_object(gathered, (kjt.values().cpu(), kjt.lengths().cpu()), group=ctx.pg)
            from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

            kjts = [KeyedJaggedTensor(keys=kjt.keys(), values=v.to(ctx.device), lengths=l.to(ctx.device)) for v, l in gathered]
            # d(mean of logits) / d(pooled row) is the same for every sample; gradients are averaged over the ranks
            grad_row = (over_w[0] / B / world_size).to(torch.bfloat16).float()
            _oracle_update(full, state, kjts, B, mean, grad_row, 0.1, 1e-8, world_size)
        torch.cuda.synchronize()
        check_all()
        assert _sharded_ebc(fused)._engine is not None, "the fused sparse engine must be active on a 2-GPU node"
        for name, v in fused.state_dict().items():
            if not hasattr(v, "local_shards"):
                continue
            ti = int(name.split(".t")[-1].split(".")[0])
            for sh in v.local_shards():
                ro, co = sh.metadata.shard_offsets
                rs, cs = sh.metadata.shard_sizes
                torch.testing.assert_close(sh.tensor, full[ti][ro: ro + rs, co: co + cs], rtol=2e-2, atol=2e-4)


@pytest.mark.parametrize("pooling_name", ["SUM", "MEAN"])
def test_engine_matches_unsharded_oracle(pooling_name):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    run_multi_process(_run, world_size=2, timeout_s=120, pooling_name=pooling_name)


def _run_late(rank, world_size):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import faulthandler

    faulthandler.dump_traceback_later(100, exit=True)
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
    run_multi_process(_run_late, world_size=2, timeout_s=120)
