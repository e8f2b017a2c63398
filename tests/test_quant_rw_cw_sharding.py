"""Row-wise and column-wise placement of quantized pooled tables must reproduce the unsharded quantized module exactly (the shards
hold the very same quantized bytes)."""
import pytest
import torch

from torchrec_b200.distributed.quant_embeddingbag import ShardedQuantEmbeddingBagCollection
from torchrec_b200.distributed.types import ParameterSharding, ShardingEnv
from torchrec_b200.modules.embedding_configs import DataType, EmbeddingBagConfig, PoolingType
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
from torchrec_b200.quant.embedding_modules import EmbeddingBagCollection as QEBC
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


def _quantized(dtype: DataType, weighted: bool):
    torch.manual_seed(0)
    tables = [
        EmbeddingBagConfig(name="tw", embedding_dim=16, num_embeddings=30, feature_names=["f_tw"], pooling=PoolingType.SUM),
        EmbeddingBagConfig(name="rw_sum", embedding_dim=16, num_embeddings=37, feature_names=["f_rs", "f_rs2"], pooling=PoolingType.SUM),
        EmbeddingBagConfig(name="rw_mean", embedding_dim=16, num_embeddings=10, feature_names=["f_rm"], pooling=PoolingType.SUM if weighted else PoolingType.MEAN),
        EmbeddingBagConfig(name="cw", embedding_dim=48, num_embeddings=25, feature_names=["f_cw"], pooling=PoolingType.SUM),
    ]
    ebc = EmbeddingBagCollection(tables=tables, is_weighted=weighted)
    for t in tables:
        t.data_type = dtype
    return QEBC.from_float(_with_qconfig(ebc, dtype)), tables


def _with_qconfig(ebc, dtype):
    import torch.ao.quantization as tq

    from torchrec_b200.quant.embedding_modules import QuantConfig

    qd = {DataType.INT8: torch.qint8, DataType.INT4: torch.quint4x2}[dtype]
    ebc.qconfig = QuantConfig(activation=tq.PlaceholderObserver.with_args(dtype=torch.float), weight=tq.PlaceholderObserver.with_args(dtype=qd))
    return ebc


def _kjt(tables, B, weighted, seed):
    g = torch.Generator().manual_seed(seed)
    keys, lens, vals = [], [], []
    for t in tables:
        for f in t.feature_names:
            l = torch.randint(0, 5, (B,), generator=g)
            keys.append(f)
            lens.append(l)
            vals.append(torch.randint(0, t.num_embeddings, (int(l.sum()),), generator=g))
    v = torch.cat(vals)
    return KeyedJaggedTensor(keys=keys, values=v, lengths=torch.cat(lens), weights=torch.rand(v.numel(), generator=g) if weighted else None)


@pytest.mark.parametrize("dtype", [DataType.INT8, DataType.INT4])
@pytest.mark.parametrize("weighted", [False, True])
def test_rw_cw_match_unsharded(dtype, weighted):
    q, tables = _quantized(dtype, weighted)
    W = 3
    plan = {
        "tw": ParameterSharding(sharding_type="table_wise", compute_kernel="quant", ranks=[1]),
        "rw_sum": ParameterSharding(sharding_type="row_wise", compute_kernel="quant", ranks=list(range(W))),
        "rw_mean": ParameterSharding(sharding_type="row_wise", compute_kernel="quant", ranks=list(range(W))),
        "cw": ParameterSharding(sharding_type="column_wise", compute_kernel="quant", ranks=[2, 0, 1]),
    }
    sharded = ShardedQuantEmbeddingBagCollection(q, plan, ShardingEnv.from_local(world_size=W, rank=0), device=torch.device("cpu"))
    for seed in range(3):
        kjt = _kjt(tables, 6, weighted, seed)
        # key order of the request differs from table order
        kjt = kjt.permute([4, 0, 3, 1, 2])
        want, got = q(kjt), sharded(kjt)
        assert want.keys() == got.keys() and want.length_per_key() == got.length_per_key()
        torch.testing.assert_close(got.values(), want.values(), rtol=1e-5, atol=1e-6)
    names = list(sharded.sharded_parameter_names())
    assert "_rw_shards.2.embedding_bags.rw_sum.weight" in names and "_cw_shards.0.embedding_bags.cw.weight" in names and "_shards.1.embedding_bags.tw.weight" in names


def test_cw_on_one_device_twice_is_rejected():
    q, _ = _quantized(DataType.INT8, False)
    plan = {n: ParameterSharding(sharding_type="table_wise", compute_kernel="quant", ranks=[0]) for n in ("tw", "rw_sum", "rw_mean")}
    plan["cw"] = ParameterSharding(sharding_type="column_wise", compute_kernel="quant", ranks=[0, 0])
    with pytest.raises(ValueError):
        ShardedQuantEmbeddingBagCollection(q, plan, ShardingEnv.from_local(world_size=2, rank=0), device=torch.device("cpu"))


@pytest.mark.parametrize("need_indices", [False, True])
def test_sequence_rw_cw_match_unsharded(need_indices):
    from torchrec_b200.distributed.quant_embedding import ShardedQuantEmbeddingCollection
    from torchrec_b200.modules.embedding_configs import EmbeddingConfig
    from torchrec_b200.modules.embedding_modules import EmbeddingCollection
    from torchrec_b200.quant.embedding_modules import EmbeddingCollection as QEC

    torch.manual_seed(1)
    tables = [EmbeddingConfig(name="tw", embedding_dim=24, num_embeddings=30, feature_names=["f_tw"]),
              EmbeddingConfig(name="rw", embedding_dim=24, num_embeddings=41, feature_names=["f_r1", "f_r2"]),
              EmbeddingConfig(name="cw3", embedding_dim=24, num_embeddings=25, feature_names=["f_c3"]),
              EmbeddingConfig(name="cw2", embedding_dim=24, num_embeddings=19, feature_names=["f_c2"])]
    ec = EmbeddingCollection(tables=tables, need_indices=need_indices)
    q = QEC.from_float(_with_qconfig(ec, DataType.INT8))
    W = 3
    plan = {"tw": ParameterSharding(sharding_type="table_wise", compute_kernel="quant", ranks=[2]),
            "rw": ParameterSharding(sharding_type="row_wise", compute_kernel="quant", ranks=list(range(W))),
            "cw3": ParameterSharding(sharding_type="column_wise", compute_kernel="quant", ranks=[1, 2, 0]),
            "cw2": ParameterSharding(sharding_type="column_wise", compute_kernel="quant", ranks=[0, 2])}
    sharded = ShardedQuantEmbeddingCollection(q, plan, ShardingEnv.from_local(world_size=W, rank=0), device=torch.device("cpu"))
    for seed in range(3):
        kjt = _kjt(tables, 5, False, seed).permute([3, 0, 4, 2, 1])
        want, got = q(kjt), sharded(kjt)
        assert sorted(want) == sorted(got)
        for k in want:
            torch.testing.assert_close(got[k].values(), want[k].values(), rtol=1e-5, atol=1e-6)
            assert torch.equal(got[k].lengths(), want[k].lengths())
            if need_indices:
                assert torch.equal(got[k].weights(), want[k].weights())


def test_weight_specs_of_rw_and_cw_shards():
    from torchrec_b200.distributed.quant_state import sharded_tbes_weights_spec

    q, _ = _quantized(DataType.INT8, False)
    W = 3
    plan = {"tw": ParameterSharding(sharding_type="table_wise", compute_kernel="quant", ranks=[1]),
            "rw_sum": ParameterSharding(sharding_type="row_wise", compute_kernel="quant", ranks=list(range(W))),
            "rw_mean": ParameterSharding(sharding_type="table_wise", compute_kernel="quant", ranks=[0]),
            "cw": ParameterSharding(sharding_type="column_wise", compute_kernel="quant", ranks=[2, 0, 1])}
    sharded = ShardedQuantEmbeddingBagCollection(q, plan, ShardingEnv.from_local(world_size=W, rank=0), device=torch.device("cpu"))
    spec = sharded_tbes_weights_spec(torch.nn.ModuleDict({"ebc": sharded}))
    by_fqn = {}
    for k, v in spec.items():
        if k.endswith(".weight"):
            by_fqn.setdefault(v.fqn, []).append(v)
    rw = sorted(by_fqn["ebc.embedding_bags.rw_sum.weight"], key=lambda w: w.shard_offsets[0])
    assert [(w.shard_offsets, w.shard_sizes) for w in rw] == [([0, 0], [13, 16]), ([13, 0], [13, 16]), ([26, 0], [11, 16])] and rw[0].sharding_type == "row_wise"
    cw = sorted(by_fqn["ebc.embedding_bags.cw.weight"], key=lambda w: w.shard_offsets[1])
    assert [(w.shard_offsets, w.shard_sizes) for w in cw] == [([0, 0], [25, 16]), ([0, 16], [25, 16]), ([0, 32], [25, 16])] and cw[0].sharding_type == "column_wise"
    assert by_fqn["ebc.embedding_bags.tw.weight"][0].shard_sizes == [30, 16]


def test_shard_quant_model_honours_constraints():
    from torchrec_b200.distributed.planner import ParameterConstraints
    from torchrec_b200.inference.modules import shard_quant_model

    q, tables = _quantized(DataType.INT8, False)
    holder = torch.nn.Sequential(q)
    kjt = _kjt(tables, 4, False, 5)
    want = q(kjt).values().clone()
    sharded, plan = shard_quant_model(holder, world_size=3, compute_device="cpu",
                                      constraints={"rw_sum": ParameterConstraints(sharding_types=["row_wise"]), "cw": ParameterConstraints(sharding_types=["column_wise"])})
    p = plan.plan["0"]
    assert p["rw_sum"].sharding_type == "row_wise" and p["rw_sum"].ranks == [0, 1, 2]
    assert p["cw"].sharding_type == "column_wise" and len(p["cw"].ranks) == 3 and p["tw"].sharding_type == "table_wise"
    torch.testing.assert_close(sharded(kjt).values(), want, rtol=1e-5, atol=1e-6)


def test_shard_quant_model_splits_tables_that_do_not_fit():
    from torchrec_b200.inference.modules import shard_quant_model

    q, tables = _quantized(DataType.INT8, False)
    kjt = _kjt(tables, 4, False, 9)
    want = q(kjt).values().clone()
    sizes = {n: h.weight.numel() for n, h in q.embedding_bags.items()}
    # room for the largest table's half only: it must be split, the small ones still go whole
    sharded, plan = shard_quant_model(torch.nn.Sequential(q), world_size=2, compute_device="cpu", device_memory_size=max(sizes.values()) - 1)
    kinds = {n: ps.sharding_type for n, ps in plan.plan["0"].items()}
    biggest = max(sizes, key=sizes.get)
    assert kinds[biggest] == "row_wise"
    torch.testing.assert_close(sharded(kjt).values(), want, rtol=1e-5, atol=1e-6)
    # with room to spare everything stays table-wise
    q2, _ = _quantized(DataType.INT8, False)
    _, roomy = shard_quant_model(torch.nn.Sequential(q2), world_size=2, compute_device="cpu", device_memory_size=10 * sum(sizes.values()))
    assert {ps.sharding_type for ps in roomy.plan["0"].values()} == {"table_wise"}


def test_sharded_state_reassembles_the_unsharded_tables():
    """The checkpoint view of a sharded serving module: pieces carry offsets that put the unsharded packed table back together."""
    q, tables = _quantized(DataType.INT8, False)
    W = 3
    plan = {"tw": ParameterSharding(sharding_type="table_wise", compute_kernel="quant", ranks=[1]),
            "rw_sum": ParameterSharding(sharding_type="row_wise", compute_kernel="quant", ranks=list(range(W))),
            "rw_mean": ParameterSharding(sharding_type="row_wise", compute_kernel="quant", ranks=list(range(W))),
            "cw": ParameterSharding(sharding_type="column_wise", compute_kernel="quant", ranks=[2, 0, 1])}
    sharded = ShardedQuantEmbeddingBagCollection(q, plan, ShardingEnv.from_local(world_size=W, rank=0), device=torch.device("cpu"))
    sd = sharded.sharded_state_dict(prefix="m.")
    for t in tables:
        packed = q.embedding_bags[t.name].weight
        payload = t.embedding_dim  # int8: one byte per element
        got = sd[f"m.embedding_bags.{t.name}.weight"]
        tail = sd[f"m.embedding_bags.{t.name}.weight_qscalebias"]
        if t.name == "tw":
            assert torch.equal(got, packed[:, :payload]) and torch.equal(tail, packed[:, payload:])
            continue
        rebuilt = torch.zeros(t.num_embeddings, payload, dtype=torch.uint8)
        for sh in got.local_shards():
            (r0, c0), (nr, nc) = sh.metadata.shard_offsets, sh.metadata.shard_sizes
            rebuilt[r0: r0 + nr, c0: c0 + nc] = sh.tensor
        assert torch.equal(rebuilt, packed[:, :payload]), t.name
        for sh in tail.local_shards():
            r0, nr = sh.metadata.shard_offsets[0], sh.metadata.shard_sizes[0]
            assert torch.equal(sh.tensor, packed[r0: r0 + nr, payload:])


def test_sharded_quant_fp_ebc_and_mc_ec_match_unsharded():
    import torch.ao.quantization as tq

    from torchrec_b200.distributed.quant_embedding import QuantManagedCollisionEmbeddingCollectionSharder, ShardedQuantManagedCollisionEmbeddingCollection
    from torchrec_b200.distributed.quant_embeddingbag import QuantFeatureProcessedEmbeddingBagCollectionSharder, ShardedQuantFeatureProcessedEmbeddingBagCollection
    from torchrec_b200.modules.embedding_configs import EmbeddingConfig, QuantConfig
    from torchrec_b200.modules.embedding_modules import EmbeddingCollection
    from torchrec_b200.modules.feature_processor_ import PositionWeightedModuleCollection
    from torchrec_b200.modules.fp_embedding_modules import FeatureProcessedEmbeddingBagCollection
    from torchrec_b200.modules.mc_embedding_modules import ManagedCollisionEmbeddingCollection
    from torchrec_b200.modules.mc_modules import LFU_EvictionPolicy, ManagedCollisionCollection, MCHManagedCollisionModule
    from torchrec_b200.quant.embedding_modules import FeatureProcessedEmbeddingBagCollection as QFPEBC
    from torchrec_b200.quant.embedding_modules import QuantManagedCollisionEmbeddingCollection as QMCEC

    qconfig = QuantConfig(activation=tq.PlaceholderObserver.with_args(dtype=torch.float), weight=tq.PlaceholderObserver.with_args(dtype=torch.qint8))
    torch.manual_seed(2)
    tables = [EmbeddingBagConfig(name="a", embedding_dim=16, num_embeddings=33, feature_names=["fa"], pooling=PoolingType.SUM),
              EmbeddingBagConfig(name="b", embedding_dim=32, num_embeddings=21, feature_names=["fb"], pooling=PoolingType.SUM)]
    fp = PositionWeightedModuleCollection({"fa": 6, "fb": 6})
    with torch.no_grad():
        for p in fp.parameters():
            p.uniform_(0.5, 1.5)
    fp_ebc = FeatureProcessedEmbeddingBagCollection(EmbeddingBagCollection(tables, is_weighted=True), fp)
    fp_ebc.qconfig = qconfig
    q = QFPEBC.from_float(fp_ebc)
    plan = {"a": ParameterSharding(sharding_type="row_wise", compute_kernel="quant", ranks=[0, 1]),
            "b": ParameterSharding(sharding_type="column_wise", compute_kernel="quant", ranks=[1, 0])}
    sharder = QuantFeatureProcessedEmbeddingBagCollectionSharder()
    assert sharder.module_type is QFPEBC
    sharded = sharder.shard(q, plan, ShardingEnv.from_local(world_size=2, rank=0), torch.device("cpu"))
    assert isinstance(sharded, ShardedQuantFeatureProcessedEmbeddingBagCollection)
    kjt = _kjt(tables, 7, False, 3)
    torch.testing.assert_close(sharded(kjt).values(), q(kjt).values(), rtol=1e-5, atol=1e-6)

    cfg = EmbeddingConfig(name="t", num_embeddings=8, embedding_dim=16, feature_names=["f"])
    ec = EmbeddingCollection(tables=[cfg])
    mcc = ManagedCollisionCollection({"t": MCHManagedCollisionModule(zch_size=8, device=torch.device("cpu"), eviction_policy=LFU_EvictionPolicy(), eviction_interval=1)}, [cfg])
    mc_ec = ManagedCollisionEmbeddingCollection(ec, mcc, return_remapped_features=True)
    raw = KeyedJaggedTensor.from_lengths_sync(keys=["f"], values=torch.tensor([1000, 2000, 1000, 3000, 1000, 4000]), lengths=torch.tensor([2, 4]))
    mc_ec.train()
    for _ in range(3):
        mc_ec(raw)
    mc_ec.eval()
    mc_ec.qconfig = qconfig
    qmc = QMCEC.from_float(mc_ec)
    sharded_mc = QuantManagedCollisionEmbeddingCollectionSharder().shard(
        qmc, {"t": ParameterSharding(sharding_type="row_wise", compute_kernel="quant", ranks=[0, 1])}, ShardingEnv.from_local(world_size=2, rank=0), torch.device("cpu"))
    assert isinstance(sharded_mc, ShardedQuantManagedCollisionEmbeddingCollection)
    (want, want_ids), (got, got_ids) = qmc(raw), sharded_mc(raw)
    assert torch.equal(want_ids.values(), got_ids.values())
    torch.testing.assert_close(got["f"].values(), want["f"].values(), rtol=1e-5, atol=1e-6)
