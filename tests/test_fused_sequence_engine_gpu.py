"""Fused sequence engine on ONE GPU: several virtual ranks, each with its own shard kernels and buffers in local memory.

Every phase is run for all virtual ranks before the next phase starts, so no kernel ever waits for a later launch.  The
oracle is plain fp32 torch on the unsharded tables: an index into the table for the rows, and a row-wise Adagrad written
out in torch for the update.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _build(world, plan_kinds, dim, rows, stage_dtype=torch.float32, grad_dtype=torch.float32):
    from torchrec_b200.distributed.embedding import EmbeddingCollectionSharder, ShardedEmbeddingCollection, create_embedding_sharding
    from torchrec_b200.distributed.fused_sequence_engine import FusedSequenceEngine
    from torchrec_b200.distributed.peer_memory import EmulatedPeerGroup
    from torchrec_b200.distributed.sharding_plan import column_wise, construct_module_sharding_plan, row_wise, table_wise
    from torchrec_b200.distributed.types import ShardingEnv
    from torchrec_b200.modules.embedding_configs import EmbeddingConfig
    from torchrec_b200.modules.embedding_modules import EmbeddingCollection
    from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward
    from torchrec_b200.optim.rowwise_adagrad import RowWiseAdagrad

    dev = torch.device("cuda:0")
    tables = [EmbeddingConfig(name=f"t{i}", embedding_dim=dim, num_embeddings=r, feature_names=[f"f{i}"]) for i, r in enumerate(rows)]
    ec = EmbeddingCollection(tables=tables, device=torch.device("meta"))
    apply_optimizer_in_backward(RowWiseAdagrad, ec.parameters(), {"lr": 0.05, "eps": 1e-8})
    gens = {}
    for i, kind in enumerate(plan_kinds):
        if kind == "tw":
            gens[f"t{i}"] = table_wise(rank=i % world)
        elif kind == "rw":
            gens[f"t{i}"] = row_wise()
        else:
            gens[f"t{i}"] = column_wise(ranks=[(i + k) % world for k in range(2)])
    plan = construct_module_sharding_plan(ec, gens, sharder=EmbeddingCollectionSharder(), local_size=world, world_size=world, device_type="cuda")
    emu = EmulatedPeerGroup(world, dev)
    engines, lookups_all = [], []
    torch.manual_seed(0)
    full = [torch.randn(r, dim, device=dev) * 0.1 for r in rows]
    for rank in range(world):
        env = ShardingEnv(world, rank, None)
        infos = ShardedEmbeddingCollection.create_grouped_sharding_infos(ec, plan, {})
        shardings = [create_embedding_sharding(st, v, env, dev) for st, v in infos.items()]
        lookups = [s.create_lookup() for s in shardings]
        for lk in lookups:
            for emb in lk.emb_modules:
                for t, w in zip(emb.config.embedding_tables, emb.split_embedding_weights()):
                    ro, co = t.local_metadata.shard_offsets
                    rs, cs = t.local_metadata.shard_sizes
                    w.copy_(full[int(t.name[1:])][ro: ro + rs, co: co + cs])
        engines.append(FusedSequenceEngine(emu.view(rank), tables, shardings, lookups, torch.float32, stage_dtype, grad_dtype))
        lookups_all.append(lookups)
    return tables, engines, lookups_all, full


def _kjt(tables, B, max_len, seed, idx_dtype=torch.int64):
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    g = torch.Generator().manual_seed(seed)
    keys = [f for t in tables for f in t.feature_names]
    lengths = torch.randint(0, max_len + 1, (len(keys) * B,), generator=g, dtype=torch.int32)
    vals = []
    for k, t in enumerate(tables):
        n = int(lengths[k * B:(k + 1) * B].sum())
        vals.append(torch.randint(0, t.num_embeddings, (n,), generator=g))
    return KeyedJaggedTensor(keys=keys, values=torch.cat(vals).to(idx_dtype).cuda(), lengths=lengths.cuda())


def _table_of_value(tables, kjt, B):
    """Table index of every id of the KJT (ids are key-major)."""
    off = kjt.offsets().long().cpu()
    per_key = [int(off[(k + 1) * B] - off[k * B]) for k in range(len(tables))]
    return torch.repeat_interleave(torch.arange(len(tables)), torch.tensor(per_key)).cuda()


def _oracle_rows(tables, full, kjt, B):
    tbl = _table_of_value(tables, kjt, B)
    vals = kjt.values().long()
    out = torch.zeros(vals.numel(), full[0].shape[1], device="cuda")
    for ti in range(len(tables)):
        m = tbl == ti
        out[m] = full[ti][vals[m]]
    return out


def _run_step(engines, kjts, grads=None):
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
    (1, ["tw", "tw"], torch.int64),
    (2, ["tw", "tw", "tw"], torch.int64),
    (2, ["rw", "tw", "cw"], torch.int32),
    (4, ["rw", "rw", "tw", "cw", "tw"], torch.int64),
])
def test_rows_match_unsharded(world, kinds, idx_dtype):
    rows = [1000, 37, 5000, 64, 3][: len(kinds)]
    tables, engines, _, full = _build(world, kinds, 32, rows)
    B = 300  # two chunks of 256 bags, the second one partial
    for step in range(2):  # the second step reuses buffers, flags and epochs
        kjts = [_kjt(tables, B, 7, 10 * step + r, idx_dtype=idx_dtype) for r in range(world)]
        outs = _run_step(engines, kjts)
        for r in range(world):
            torch.testing.assert_close(outs[r], _oracle_rows(tables, full, kjts[r], B), rtol=0, atol=0)


def test_half_precision_exchange():
    tables, engines, _, full = _build(2, ["rw", "tw"], 64, [800, 50], stage_dtype=torch.float16, grad_dtype=torch.bfloat16)
    kjts = [_kjt(tables, 128, 6, r) for r in range(2)]
    outs = _run_step(engines, kjts)
    for r in range(2):
        torch.testing.assert_close(outs[r], _oracle_rows(tables, full, kjts[r], 128), rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("world", [1, 2])
def test_backward_updates_match_rowwise_adagrad(world):
    kinds = ["rw", "tw", "cw"]
    dim, rows = 16, [200, 37, 64]
    tables, engines, lookups_all, full = _build(world, kinds, dim, rows)
    B = 96
    kjts = [_kjt(tables, B, 6, r) for r in range(world)]
    torch.manual_seed(3)
    grads = [torch.randn(k.values().numel(), dim, device="cuda") for k in kjts]
    _run_step(engines, kjts, grads)
    for ti, t in enumerate(tables):
        gsum = torch.zeros_like(full[ti])
        for r in range(world):
            m = _table_of_value(tables, kjts[r], B) == ti
            gsum.index_add_(0, kjts[r].values().long()[m], grads[r][m])
        touched = gsum.abs().sum(1) > 0
        # column-wise shards keep one row-wise state per shard: the oracle does the same per column block
        blocks = [(0, dim)] if kinds[ti] != "cw" else [(0, dim // 2), (dim // 2, dim)]
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


def test_sharded_embedding_collection_uses_the_engine_on_one_rank():
    """The module-level path: ``ShardedEmbeddingCollection`` on a one-rank environment routes through the engine and returns
    the same per-feature jagged tensors as the unsharded module; its backward updates the tables in place."""
    import tempfile

    import torch.distributed as dist

    dev = torch.device("cuda:0")
    own_group = not dist.is_initialized()
    if own_group:  # the module builds its (unused) library output dists against a process group
        dist.init_process_group("gloo", store=dist.FileStore(tempfile.mktemp(), 1), rank=0, world_size=1)
    try:
        _one_rank_module_case(dev)
    finally:
        if own_group:
            dist.destroy_process_group()


def _one_rank_module_case(dev):
    from torchrec_b200.distributed.embedding import EmbeddingCollectionSharder
    from torchrec_b200.distributed.sharding_plan import construct_module_sharding_plan, table_wise
    from torchrec_b200.distributed.types import ShardingEnv
    from torchrec_b200.modules.embedding_configs import EmbeddingConfig
    from torchrec_b200.modules.embedding_modules import EmbeddingCollection
    from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward
    from torchrec_b200.optim.rowwise_adagrad import RowWiseAdagrad
    import torch.distributed as dist

    tables = [EmbeddingConfig(name=f"t{i}", embedding_dim=32, num_embeddings=r, feature_names=[f"f{i}"]) for i, r in enumerate([100, 2000])]
    torch.manual_seed(1)
    ec = EmbeddingCollection(tables=tables, device=dev)
    apply_optimizer_in_backward(RowWiseAdagrad, ec.parameters(), {"lr": 0.05, "eps": 1e-8})
    sharder = EmbeddingCollectionSharder()
    plan = construct_module_sharding_plan(ec, {"t0": table_wise(rank=0), "t1": table_wise(rank=0)}, sharder=sharder, local_size=1, world_size=1,
                                          device_type="cuda")
    sec = sharder.shard(ec, plan, ShardingEnv.from_process_group(dist.group.WORLD), dev)
    # the sharded module initialises its own table memory: the oracle reads it back before the step
    ref = {t.name: w.detach().clone() for lk in sec._lookups for emb in lk.emb_modules for t, w in zip(emb.config.embedding_tables, emb.split_embedding_weights())}
    kjt = _kjt(tables, 50, 5, 7)
    out = sec(kjt).wait()
    assert sec._engine_state == "on"
    off = kjt.offsets().long().cpu()
    for i in range(2):
        s, e = int(off[i * 50]), int(off[(i + 1) * 50])
        torch.testing.assert_close(out[f"f{i}"].values(), ref[f"t{i}"][kjt.values()[s:e]], rtol=0, atol=0)
        assert torch.equal(out[f"f{i}"].lengths(), kjt.lengths()[i * 50:(i + 1) * 50])
    loss = sum(jt.values().sum() for jt in out.values())
    loss.backward()
    torch.cuda.synchronize()
    w1 = [w for lk in sec._lookups for emb in lk.emb_modules for t, w in zip(emb.config.embedding_tables, emb.split_embedding_weights()) if t.name == "t1"][0]
    s, e = int(off[50]), int(off[100])
    touched = torch.unique(kjt.values()[s:e])
    assert not torch.equal(w1[touched], ref["t1"][touched])
    untouched = torch.ones(2000, dtype=torch.bool, device=dev)
    untouched[touched] = False
    assert torch.equal(w1[untouched], ref["t1"][untouched])
