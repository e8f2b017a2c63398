"""C++ dynamic-embedding library through its torch class bindings: id transformer (slot assignment, LFU/LRU
eviction order, resume after "out of slots"), parameter-server client with the in-process store (evict -> fetch round
trip, re-initialisation of unknown ids, column shards) — cf. ``test/cpp/dynamic_embedding/*.cpp`` of the reference."""
import pytest
import torch

from torchrec_b200.ops import _ext


@pytest.fixture(scope="module", autouse=True)
def _lib():
    if not _ext.has_cpu_ext():
        pytest.skip("native CPU library not built")


def test_id_transformer_assigns_slots_and_reports_new_ids():
    t = torch.classes.trb_tde.IDTransformer(4, 5, "naive")
    gids = torch.tensor([100, 7, 100, 42], dtype=torch.long)
    slots = torch.empty_like(gids)
    r = t.transform(gids, slots, 1)
    assert r.success and r.num_transformed == 4
    assert slots.tolist() == [0, 1, 0, 2]
    assert r.ids_to_fetch.tolist() == [[100, 0], [7, 1], [42, 2]]
    assert t.size() == 3
    # known ids are not reported again
    r2 = t.transform(gids, slots, 2)
    assert r2.ids_to_fetch.numel() == 0 and slots.tolist() == [0, 1, 0, 2]


def test_id_transformer_full_then_evict_and_resume():
    t = torch.classes.trb_tde.IDTransformer(3, 0, "cacheline")
    slots = torch.empty(5, dtype=torch.long)
    gids = torch.tensor([1, 2, 3, 4, 5], dtype=torch.long)
    r = t.transform(gids, slots, 1)
    assert not r.success and r.num_transformed == 3
    # id 3 was touched many more times: the frequency part of its record protects it
    for step in range(2, 40):
        t.transform(torch.tensor([3], dtype=torch.long), torch.empty(1, dtype=torch.long), step)
    ev = t.evict(2)
    assert sorted(ev[:, 0].tolist()) == [1, 2]
    r = t.transform(gids[3:], slots[3:], 50)
    assert r.success and sorted(slots[3:].tolist()) == sorted(ev[:, 1].tolist())
    assert sorted(x[0] for x in t.save().tolist()) == [3, 4, 5]


def test_lru_order_within_equal_frequency():
    t = torch.classes.trb_tde.IDTransformer(4, 5, "naive")
    for time, gid in enumerate([10, 11, 12, 13], start=1):
        t.transform(torch.tensor([gid], dtype=torch.long), torch.empty(1, dtype=torch.long), time)
    assert t.evict(2)[:, 0].tolist() == [10, 11]  # oldest first


@pytest.mark.parametrize("col_shards", [1, 2])
def test_ps_evict_fetch_round_trip(col_shards):
    rows, dim = 6, 8
    torch.manual_seed(0)
    w = torch.randn(rows, dim)
    m = torch.randn(rows)  # row-wise optimizer state
    shards = torch.classes.trb_tde.LocalShardList()
    step = dim // col_shards
    views = []
    for c in range(col_shards):
        wv = w[:, c * step:(c + 1) * step]
        views.append(wv)
        shards.append(0, c * step, rows, step, [wv, m if c == 0 else m.clone()])
    ps = torch.classes.trb_tde.PS(f"tbl{col_shards}", shards, dim, 1, f"memory://test{col_shards}", 2)
    expect_w, expect_m = w[[1, 4, 5]].clone(), m[[1, 4, 5]].clone()
    ps.evict(torch.tensor([[1001, 1], [1004, 4], [1005, 5]], dtype=torch.long))
    w.zero_(); m.zero_()
    # fetch into other slots; id 777 is unknown and gets re-initialised
    h = ps.fetch(torch.tensor([[1004, 0], [1001, 2], [1005, 3], [777, 5]], dtype=torch.long), 3, True, -0.5, 0.5)
    h.wait()
    torch.testing.assert_close(w[[2, 0, 3]], expect_w)
    torch.testing.assert_close(m[[2, 0, 3]], expect_m)
    assert w[5].abs().max() <= 0.5 and w[5].abs().sum() > 0 and float(m[5]) == 0.0
    assert w[[1, 4]].abs().sum() == 0  # untouched slots stay as they were


def test_unknown_io_type_raises():
    shards = torch.classes.trb_tde.LocalShardList()
    with pytest.raises(RuntimeError, match="no IO provider"):
        torch.classes.trb_tde.PS("t", shards, 8, 0, "nosuchstore://127.0.0.1:6379", 10)


def test_id_transformer_collection_keeps_rows_across_eviction():
    """Global ids far beyond the table size train through an 8-slot table; rows survive eviction via the store."""
    from torchrec_b200.contrib.dynamic_embedding import IDTransformerGroup
    from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig
    from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    cfg = EmbeddingBagConfig(name="t0", num_embeddings=8, embedding_dim=4, feature_names=["f0"])
    ebc = EmbeddingBagCollection([cfg])
    group = IDTransformerGroup("memory://coll", ebc, {"": [cfg]}, ps_config={"chunk_size": 3})
    first = {}
    for step in range(6):
        gids = torch.arange(step * 5, step * 5 + 6, dtype=torch.long) * 1_000_003  # 6 ids per step, overlapping by one
        kjt = KeyedJaggedTensor.from_lengths_sync(keys=["f0"], values=gids, lengths=torch.ones(6, dtype=torch.long))
        out, handles = group.transform({"": kjt})
        for h in handles:
            h.wait()
        slots = out[""].values()
        assert int(slots.max()) < 8 and int(slots.min()) >= 0
        rows = ebc.embedding_bags["t0"].weight.detach()[slots]
        for g, r in zip(gids.tolist(), rows):
            if g in first:
                torch.testing.assert_close(r, first[g])  # same row as when the id was first seen, wherever it lives now
            else:
                first[g] = r.clone()
    group.save()


def test_wrapped_dataloader_rewrites_ids_and_saves():
    """``wrap`` returns a loader whose batches carry cache rows instead of global ids; a failing source surfaces as an error."""
    import pytest
    from torchrec_b200.contrib import dynamic_embedding as tde
    from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig
    from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    cfg = EmbeddingBagConfig(name="t0", num_embeddings=8, embedding_dim=4, feature_names=["f0"])
    ebc = EmbeddingBagCollection([cfg])

    def source(n):
        for step in range(n):
            gids = torch.arange(step * 3, step * 3 + 4, dtype=torch.long) * 1_000_003
            yield torch.full((4,), float(step)), KeyedJaggedTensor.from_lengths_sync(keys=["f0"], values=gids, lengths=torch.ones(4, dtype=torch.long))

    loader, model = tde.wrap("memory://wrapped", list(source(5)), ebc, {"": [cfg]}, data_info={1: ""}, num_prefetch=2)
    assert model is ebc and len(loader) == 5
    seen = 0
    for label, kjt in loader:
        assert int(kjt.values().max()) < 8 and int(kjt.values().min()) >= 0 and float(label[0]) == seen
        model(kjt).values().sum().backward()
        seen += 1
    assert seen == 5
    tde.save(model)
    with pytest.raises(ValueError):
        tde.save(EmbeddingBagCollection([cfg]))

    def broken():
        yield from source(1)
        raise OSError("disk gone")

    bad, _ = tde.wrap("memory://wrapped2", broken(), EmbeddingBagCollection([cfg]), {"": [cfg]}, data_info={1: ""})
    it = iter(bad)
    next(it)
    with pytest.raises(RuntimeError):
        next(it)
    tl = tde.TensorList([torch.zeros(2)])
    tl.append(torch.ones(3))
    assert len(tl) == 2 and tl[1].numel() == 3


def test_cacheline_layout_agrees_with_the_naive_one():
    """Both table layouts of the native id transformer hand out the same slots for the same stream of ids."""
    import pytest
    import torch

    from torchrec_b200.contrib.dynamic_embedding.id_transformer import IDTransformer

    a = IDTransformer(64, transform_config={"type": "naive"})
    b = IDTransformer(64, transform_config={"type": "cacheline"})
    g = torch.Generator().manual_seed(0)
    for step in range(1, 6):
        ids = torch.randint(0, 40, (30,), generator=g)
        sa, sb = torch.empty_like(ids), torch.empty_like(ids)
        ra, rb = a.transform(ids, sa, step), b.transform(ids, sb, step)
        assert ra.success and rb.success and torch.equal(sa, sb) and torch.equal(ra.ids_to_fetch, rb.ids_to_fetch)
    assert len(a) == len(b)
    assert sorted(map(tuple, a.save().tolist())) == sorted(map(tuple, b.save().tolist()))
    with pytest.raises(Exception):
        IDTransformer(8, transform_config={"type": "other"})
