"""Fused sparse engine on ONE GPU: several virtual ranks, each with its own shard kernels and buffers in local memory.

Every phase (count, scatter, lookup push, finalize, gradient publish, pull + update) is run for all virtual ranks before
the next phase starts, so no kernel ever waits for a later launch.  The oracle is plain fp32 torch on the unsharded
tables: ``embedding_bag`` for the pooled output and a row-wise Adagrad written out in torch for the update.
"""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _build(world, plan_kinds, dims, rows, pooling, weighted=False, stage_dtype=torch.float32, grad_dtype=torch.float32, features_per_table=None):
    from torchrec_b200.distributed.embeddingbag import ShardedEmbeddingBagCollection, create_embedding_bag_sharding
    from torchrec_b200.distributed.fused_sparse_engine import FusedSparseEngine
    from torchrec_b200.distributed.peer_memory import EmulatedPeerGroup
    from torchrec_b200.distributed.sharding_plan import column_wise, construct_module_sharding_plan, row_wise, table_wise
    from torchrec_b200.distributed.embeddingbag import EmbeddingBagCollectionSharder
    from torchrec_b200.distributed.types import ShardingEnv
    from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig, PoolingType
    from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
    from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward
    from torchrec_b200.optim.rowwise_adagrad import RowWiseAdagrad

    dev = torch.device("cuda:0")
    tables = []
    for i, (r, d) in enumerate(zip(rows, dims)):
        feats = [f"f{i}"] if not features_per_table else [f"f{i}_{k}" for k in range(features_per_table[i])]
        tables.append(EmbeddingBagConfig(name=f"t{i}", embedding_dim=d, num_embeddings=r, feature_names=feats,
                                         pooling=PoolingType.MEAN if pooling[i] == "mean" else PoolingType.SUM))
    ebc = EmbeddingBagCollection(tables=tables, device=torch.device("meta"), is_weighted=weighted)
    apply_optimizer_in_backward(RowWiseAdagrad, ebc.parameters(), {"lr": 0.05, "eps": 1e-8})
    gens = {}
    for i, kind in enumerate(plan_kinds):
        if kind == "tw":
            gens[f"t{i}"] = table_wise(rank=i % world)
        elif kind == "rw":
            gens[f"t{i}"] = row_wise()
        else:
            gens[f"t{i}"] = column_wise(ranks=[(i + k) % world for k in range(2)])
    plan = construct_module_sharding_plan(ebc, gens, sharder=EmbeddingBagCollectionSharder(), local_size=world, world_size=world, device_type="cuda")
    emu = EmulatedPeerGroup(world, dev)
    engines, lookups_all = [], []
    torch.manual_seed(0)
    full = [torch.randn(r, d, device=dev) * 0.1 for r, d in zip(rows, dims)]
    for rank in range(world):
        env = ShardingEnv(world, rank, None)
        infos = ShardedEmbeddingBagCollection.create_grouped_sharding_infos(ebc, plan, "embedding_bags.", {})
        shardings = [create_embedding_bag_sharding(v, env, dev, permute_embeddings=True) for v in infos.values()]
        lookups = [s.create_lookup() for s in shardings]
        for lk in lookups:
            for emb in lk.emb_modules:
                for t, w in zip(emb.config.embedding_tables, emb.split_embedding_weights()):
                    ro, co = t.local_metadata.shard_offsets
                    rs, cs = t.local_metadata.shard_sizes
                    w.copy_(full[int(t.name[1:])][ro: ro + rs, co: co + cs])
        engines.append(FusedSparseEngine(emu.view(rank), tables, shardings, lookups, torch.float32, stage_dtype, grad_dtype))
        lookups_all.append(lookups)
    return tables, engines, lookups_all, full


def _kjt(tables, B, max_len, seed, weighted=False, idx_dtype=torch.int64):
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    g = torch.Generator().manual_seed(seed)
    keys = [f for t in tables for f in t.feature_names]
    rows = [t.num_embeddings for t in tables for _ in t.feature_names]
    lengths = torch.randint(0, max_len + 1, (len(keys) * B,), generator=g, dtype=torch.int32)
    vals = []
    for k, r in enumerate(rows):
        n = int(lengths[k * B:(k + 1) * B].sum())
        vals.append(torch.randint(0, r, (n,), generator=g))
    values = torch.cat(vals).to(idx_dtype)
    w = torch.rand(values.numel(), generator=g) if weighted else None
    return KeyedJaggedTensor(keys=keys, values=values.cuda(), lengths=lengths.cuda(), weights=None if w is None else w.cuda())


def _oracle_forward(tables, full, kjt, B):
    outs = []
    off = kjt.offsets().long().cpu()
    vals = kjt.values().long()
    w = kjt.weights_or_none()
    k = 0
    for ti, t in enumerate(tables):
        for _ in t.feature_names:
            s, e = int(off[k * B]), int(off[(k + 1) * B])
            o = (off[k * B:(k + 1) * B] - s).cuda()
            if e > s:
                res = torch.nn.functional.embedding_bag(vals[s:e], full[ti], o, mode="sum", per_sample_weights=None if w is None else w[s:e])
            else:
                res = torch.zeros(B, full[ti].shape[1], device="cuda")
            if t.pooling.value == "MEAN":
                lens = (off[k * B + 1:(k + 1) * B + 1] - off[k * B:(k + 1) * B]).clamp(min=1).cuda().float()
                res = res / lens.unsqueeze(1)
            outs.append(res)
            k += 1
    return torch.cat(outs, dim=1)


def _run_step(engines, kjts, grads=None):
    W = len(engines)
    if kjts[0].stride() not in engines[0]._bufs:
        for e, k in zip(engines, kjts):
            e.prepare(k)
        for e in engines:
            e.prepare_finish()
    hs = [e.new_handle(k) for e, k in zip(engines, kjts)]
    for ph in (0, 1):
        for e, h in zip(engines, hs):
            e.phase_send(h, ph)
    for e, h in zip(engines, hs):
        e.phase_push(h, build_plans=grads is not None)
    outs = [e.phase_finalize(h) for e, h in zip(engines, hs)]
    if grads is not None:
        for e, h, g in zip(engines, hs, grads):
            e.phase_publish(h, g, 1.0)
        for e, h in zip(engines, hs):
            e.phase_pull(h)
    torch.cuda.synchronize()
    for e in engines:
        e.peer.check_error()
    return outs


@pytest.mark.parametrize("world,kinds,idx_dtype", [
    (2, ["tw", "tw", "tw"], torch.int64),
    (2, ["rw", "tw", "cw"], torch.int32),
    (4, ["rw", "rw", "tw", "cw", "tw"], torch.int64),
])
def test_forward_matches_unsharded(world, kinds, idx_dtype):
    n = len(kinds)
    dims = [16, 64, 128, 32, 8][:n]
    rows = [1000, 37, 5000, 64, 3][:n]
    tables, engines, _, full = _build(world, kinds, dims, rows, ["sum"] * n)
    B = 300  # two chunks of 256 bags, the second one partial
    for step in range(2):  # the second step reuses buffers, flags and epochs
        kjts = [_kjt(tables, B, 7, 10 * step + r, idx_dtype=idx_dtype) for r in range(world)]
        outs = _run_step(engines, kjts)
        for r in range(world):
            want = _oracle_forward(tables, full, kjts[r], B)
            torch.testing.assert_close(outs[r], want, rtol=1e-5, atol=1e-5)


def test_mean_pooling_and_weights_and_shared_table():
    tables, engines, _, full = _build(2, ["rw", "tw"], [32, 16], [500, 40], ["mean", "mean"], features_per_table=[2, 1])
    kjts = [_kjt(tables, 64, 5, r) for r in range(2)]
    outs = _run_step(engines, kjts)
    for r in range(2):
        torch.testing.assert_close(outs[r], _oracle_forward(tables, full, kjts[r], 64), rtol=1e-5, atol=1e-5)
    tables, engines, _, full = _build(2, ["rw", "tw"], [32, 16], [500, 40], ["sum", "sum"], weighted=True)
    kjts = [_kjt(tables, 64, 5, r, weighted=True) for r in range(2)]
    outs = _run_step(engines, kjts)
    for r in range(2):
        torch.testing.assert_close(outs[r], _oracle_forward(tables, full, kjts[r], 64), rtol=1e-5, atol=1e-5)


def test_half_precision_staging():
    tables, engines, _, full = _build(2, ["rw", "tw"], [64, 128], [800, 50], ["sum", "sum"], stage_dtype=torch.float16, grad_dtype=torch.bfloat16)
    kjts = [_kjt(tables, 128, 6, r) for r in range(2)]
    outs = _run_step(engines, kjts)
    for r in range(2):
        torch.testing.assert_close(outs[r], _oracle_forward(tables, full, kjts[r], 128), rtol=2e-3, atol=2e-3)


def test_backward_updates_match_rowwise_adagrad():
    world, kinds = 2, ["rw", "tw", "cw"]
    dims, rows = [16, 64, 32], [200, 37, 64]
    tables, engines, lookups_all, full = _build(world, kinds, dims, rows, ["sum"] * 3)
    B = 96
    kjts = [_kjt(tables, B, 6, r) for r in range(world)]
    torch.manual_seed(3)
    grads = [torch.randn(B, sum(dims), device="cuda") for _ in range(world)]
    _run_step(engines, kjts, grads)
    # oracle: summed gradient per table row over the global batch, then row-wise Adagrad (state = mean of squared gradient)
    col = 0
    for ti, t in enumerate(tables):
        d = dims[ti]
        gsum = torch.zeros_like(full[ti])
        for r in range(world):
            off = kjts[r].offsets().long()
            vals = kjts[r].values().long()
            k = ti
            s, e = int(off[k * B]), int(off[(k + 1) * B])
            lens = off[k * B + 1:(k + 1) * B + 1] - off[k * B:(k + 1) * B]
            bag = torch.repeat_interleave(torch.arange(B, device="cuda"), lens)
            gsum.index_add_(0, vals[s:e], grads[r][bag, col: col + d])
        touched = gsum.abs().sum(1) > 0
        # column-wise shards keep one row-wise state per shard: the oracle does the same per column block
        blocks = [(0, d)] if kinds[ti] != "cw" else [(0, d // 2), (d // 2, d)]
        want = full[ti].clone()
        for c0, c1 in blocks:
            g = gsum[:, c0:c1]
            state = g.pow(2).mean(1)
            upd = 0.05 * g / (state.sqrt() + 1e-8).unsqueeze(1)
            want[:, c0:c1] -= torch.where(touched.unsqueeze(1), upd, torch.zeros_like(upd))
        got = torch.zeros_like(full[ti])
        for lookups in lookups_all:
            for lk in lookups:
                for emb in lk.emb_modules:
                    for tt, w in zip(emb.config.embedding_tables, emb.split_embedding_weights()):
                        if tt.name == t.name:
                            ro, co = tt.local_metadata.shard_offsets
                            rs, cs = tt.local_metadata.shard_sizes
                            got[ro: ro + rs, co: co + cs] = w
        torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)
        col += d


def test_capacity_overflow_is_reported_not_written():
    tables, engines, _, full = _build(2, ["tw", "tw"], [16, 16], [100, 100], ["sum", "sum"])
    small = [_kjt(tables, 64, 1, r) for r in range(2)]
    _run_step(engines, small)  # sizes the receive buffers for about one id per bag
    big = [_kjt(tables, 64, 60, 5 + r) for r in range(2)]
    with pytest.raises(RuntimeError, match="receive buffer"):
        _run_step(engines, big)


def test_wait_that_runs_out_returns_and_poisons_the_output():
    """Rank 1 never sends: rank 0's bounded waits give up after about a millisecond, the kernels return, the error word names
    the missing rank and the output is NaN."""
    from torchrec_b200.distributed.peer_memory import EmulatedPeerGroup

    tables, engines, _, full = _build(2, ["tw", "tw"], [16, 16], [100, 100], ["sum", "sum"])
    kjts = [_kjt(tables, 32, 3, r) for r in range(2)]
    _run_step(engines, kjts)
    e0 = engines[0]
    e0.peer.wait_cycles = 2_000_000  # about 1 ms of SM clock
    h = e0.new_handle(kjts[0])
    e0.phase_send(h, 0)
    e0.phase_send(h, 1)   # waits for rank 1's sizes, which never come
    e0.phase_push(h, build_plans=False)
    out = e0.phase_finalize(h)
    torch.cuda.synchronize()
    assert torch.isnan(out).all()
    with pytest.raises(RuntimeError, match="rank 1"):
        e0.peer.check_error()
