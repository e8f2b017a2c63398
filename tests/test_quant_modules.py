"""Quantized embedding modules against the float modules they were converted from (cf. ``torchrec/quant/tests``)."""
import pytest
import torch

from torchrec_b200.modules.embedding_configs import DataType, EmbeddingBagConfig, EmbeddingConfig, PoolingType, QuantConfig
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection, EmbeddingCollection
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


def _qconfig(dtype):
    import torch.ao.quantization as q

    return QuantConfig(activation=q.PlaceholderObserver.with_args(dtype=torch.float), weight=q.PlaceholderObserver.with_args(dtype=dtype))


def _kjt(keys, rows, B=9, seed=0):
    g = torch.Generator().manual_seed(seed)
    lens, vals = [], []
    for r in rows:
        l = torch.randint(0, 5, (B,), generator=g)
        lens.append(l); vals.append(torch.randint(0, r, (int(l.sum()),), generator=g))
    return KeyedJaggedTensor.from_lengths_sync(keys=keys, values=torch.cat(vals), lengths=torch.cat(lens))


@pytest.mark.parametrize("dtype,tol", [(torch.quint8, 0.05), (torch.quint4x2, 0.6), (torch.float16, 5e-3)])
def test_quant_ebc_matches_float(dtype, tol):
    from torchrec_b200.quant.embedding_modules import EmbeddingBagCollection as QEBC

    tables = [EmbeddingBagConfig(name="t0", num_embeddings=40, embedding_dim=16, feature_names=["f0", "f1"], pooling=PoolingType.SUM),
              EmbeddingBagConfig(name="t1", num_embeddings=30, embedding_dim=32, feature_names=["f2"], pooling=PoolingType.MEAN),
              EmbeddingBagConfig(name="t2", num_embeddings=20, embedding_dim=16, feature_names=["f3"], pooling=PoolingType.SUM)]
    ebc = EmbeddingBagCollection(tables)
    ebc.qconfig = _qconfig(dtype)
    q = QEBC.from_float(ebc)
    kjt = _kjt(["f0", "f1", "f2", "f3"], [40, 40, 30, 20])
    ref, out = ebc(kjt), q(kjt)
    assert out.keys() == ref.keys() and out.length_per_key() == ref.length_per_key()
    torch.testing.assert_close(out.values(), ref.values().detach(), rtol=0, atol=tol)
    # state dict: packed tables under the float module's keys; optional split into payload + scale/bias
    sd = q.state_dict()
    assert set(sd) == {"embedding_bags.t0.weight", "embedding_bags.t1.weight", "embedding_bags.t2.weight"}
    assert sd["embedding_bags.t0.weight"].dtype == torch.uint8
    q2 = QEBC(q.embedding_bag_configs(), False, torch.device("cpu"))
    q2.load_state_dict(sd)
    torch.testing.assert_close(q2(kjt).values(), out.values())


def test_quant_state_dict_split_scale_bias():
    from torchrec_b200.quant.embedding_modules import EmbeddingBagCollection as QEBC, quant_prep_enable_quant_state_dict_split_scale_bias

    ebc = EmbeddingBagCollection([EmbeddingBagConfig(name="t0", num_embeddings=10, embedding_dim=8, feature_names=["f0"])])
    ebc.qconfig = _qconfig(torch.quint8)
    quant_prep_enable_quant_state_dict_split_scale_bias(ebc)
    sd = QEBC.from_float(ebc).state_dict()
    assert sd["embedding_bags.t0.weight"].shape == (10, 8)
    assert sd["embedding_bags.t0.weight_qscale"].shape == (10,) and sd["embedding_bags.t0.weight_qbias"].dtype == torch.float16
    recon = sd["embedding_bags.t0.weight"].float() * sd["embedding_bags.t0.weight_qscale"].float().unsqueeze(1) + sd["embedding_bags.t0.weight_qbias"].float().unsqueeze(1)
    torch.testing.assert_close(recon, ebc.embedding_bags["t0"].weight.detach(), rtol=0, atol=0.02)


def test_quant_ec_matches_float():
    from torchrec_b200.quant.embedding_modules import EmbeddingCollection as QEC

    tables = [EmbeddingConfig(name="t0", num_embeddings=40, embedding_dim=16, feature_names=["f0"]),
              EmbeddingConfig(name="t1", num_embeddings=30, embedding_dim=16, feature_names=["f1", "f2"])]
    ec = EmbeddingCollection(tables, need_indices=True)
    ec.qconfig = _qconfig(torch.quint8)
    q = QEC.from_float(ec)
    kjt = _kjt(["f0", "f1", "f2"], [40, 30, 30])
    ref, out = ec(kjt), q(kjt)
    assert out.keys() == ref.keys()
    for k in ref:
        torch.testing.assert_close(out[k].values(), ref[k].values().detach(), rtol=0, atol=0.02)
        assert torch.equal(out[k].lengths(), ref[k].lengths())
        assert torch.equal(out[k].weights(), ref[k].weights())


@pytest.mark.gpu
@pytest.mark.parametrize("bits", [32, 16, 8, 4, 2])
@pytest.mark.parametrize("pooling", [0, 1, 2])
def test_qtbe_kernel_matches_cpu(bits, pooling):
    from torchrec_b200.modules.embedding_configs import PoolingMode
    from torchrec_b200.ops.qtbe import QuantTableBatchedEmbeddingBags
    from torchrec_b200.ops.quant_ops import quantize_rowwise_nbit

    torch.manual_seed(bits + pooling)
    D = 256 if pooling != 2 else 64
    specs = [(300, D if pooling == 2 else 64, bits), (50, D, bits)]
    ftm = [0, 1, 1]
    cpu = QuantTableBatchedEmbeddingBags(specs, ftm, PoolingMode(pooling), torch.float32)
    for t, (r, d, b) in enumerate(specs):
        cpu.table_view(t).copy_(quantize_rowwise_nbit(torch.randn(r, d), b))
    gpu = QuantTableBatchedEmbeddingBags(specs, ftm, PoolingMode(pooling), torch.float32, device="cuda")
    gpu.weights.copy_(cpu.weights)
    kjt = _kjt(["a", "b", "c"], [300, 50, 50], B=33, seed=5)
    psw = torch.rand(kjt.values().numel()) if pooling == 0 else None
    ref = cpu(kjt.values(), kjt.offsets(), psw)
    out = gpu(kjt.values().cuda(), kjt.offsets().cuda(), None if psw is None else psw.cuda())
    gpu.check_error()
    torch.testing.assert_close(out.cpu(), ref, rtol=1e-4, atol=1e-4)


def test_quant_fp_ebc_matches_float():
    """Position-weighted pooled lookups: the quantized module applies the same processors and pools with their weights."""
    from torchrec_b200.modules.feature_processor_ import PositionWeightedModuleCollection
    from torchrec_b200.modules.fp_embedding_modules import FeatureProcessedEmbeddingBagCollection
    from torchrec_b200.quant.embedding_modules import FeatureProcessedEmbeddingBagCollection as QFPEBC

    tables = [EmbeddingBagConfig(name="t0", num_embeddings=40, embedding_dim=16, feature_names=["f0"], pooling=PoolingType.SUM),
              EmbeddingBagConfig(name="t1", num_embeddings=30, embedding_dim=16, feature_names=["f1"], pooling=PoolingType.SUM)]
    torch.manual_seed(0)
    fp = PositionWeightedModuleCollection({"f0": 8, "f1": 8})
    with torch.no_grad():
        for p in fp.parameters():
            p.uniform_(0.5, 1.5)
    fp_ebc = FeatureProcessedEmbeddingBagCollection(EmbeddingBagCollection(tables, is_weighted=True), fp)
    fp_ebc.qconfig = _qconfig(torch.quint8)
    q = QFPEBC.from_float(fp_ebc)
    assert q._get_name() == "QuantFeatureProcessedEmbeddingBagCollection"
    kjt = _kjt(["f0", "f1"], [40, 30])
    ref, out = fp_ebc(kjt), q(kjt)
    assert out.keys() == ref.keys()
    torch.testing.assert_close(out.values(), ref.values().detach(), rtol=0, atol=0.08)
    with pytest.raises(AssertionError):
        QFPEBC(tables, True, torch.device("cpu"))


def test_quant_mc_ec_remaps_then_looks_up():
    """Raw ids go through the trained id map, then into the quantized table; the remapped KJT comes back with the rows."""
    from torchrec_b200.modules.mc_embedding_modules import ManagedCollisionEmbeddingCollection
    from torchrec_b200.modules.mc_modules import LFU_EvictionPolicy, ManagedCollisionCollection, MCHManagedCollisionModule
    from torchrec_b200.quant.embedding_modules import QuantManagedCollisionEmbeddingCollection

    cfg = EmbeddingConfig(name="t", num_embeddings=8, embedding_dim=16, feature_names=["f"])
    torch.manual_seed(0)
    ec = EmbeddingCollection(tables=[cfg])
    mcc = ManagedCollisionCollection({"t": MCHManagedCollisionModule(zch_size=8, device=torch.device("cpu"), eviction_policy=LFU_EvictionPolicy(), eviction_interval=1)}, [cfg])
    mc_ec = ManagedCollisionEmbeddingCollection(ec, mcc, return_remapped_features=True)
    raw = KeyedJaggedTensor.from_lengths_sync(keys=["f"], values=torch.tensor([1000, 2000, 1000, 3000, 1000]), lengths=torch.tensor([2, 3]))
    mc_ec.train()
    for _ in range(3):
        mc_ec(raw)
    mc_ec.eval()
    ref_out, ref_remapped = mc_ec(raw)
    mc_ec.qconfig = _qconfig(torch.float16)
    q = QuantManagedCollisionEmbeddingCollection.from_float(mc_ec)
    out, remapped = q(raw)
    assert torch.equal(remapped.values(), ref_remapped.values())
    torch.testing.assert_close(out["f"].values(), ref_out["f"].values().detach(), rtol=0, atol=5e-3)
    assert torch.equal(out["f"].lengths(), ref_out["f"].lengths())
    # serving does not learn: unseen ids fall back to the modulo slot and the map stays as it was
    before = q._managed_collision_collection._managed_collision_modules["t"]._mch_sorted_raw_ids.clone()
    q(KeyedJaggedTensor.from_lengths_sync(keys=["f"], values=torch.tensor([777, 778]), lengths=torch.tensor([1, 1])))
    assert torch.equal(before, q._managed_collision_collection._managed_collision_modules["t"]._mch_sorted_raw_ids)


def _forward_into_case(device):
    from torchrec_b200.modules.embedding_configs import PoolingMode
    from torchrec_b200.ops.qtbe import QuantTableBatchedEmbeddingBags
    from torchrec_b200.ops.quant_ops import quantize_rowwise_nbit

    torch.manual_seed(3)
    specs = [(300, 64, 8), (50, 128, 4)]
    ftm = [0, 1, 1]
    m = QuantTableBatchedEmbeddingBags(specs, ftm, PoolingMode.SUM, torch.float32, device=device)
    for t, (r, d, b) in enumerate(specs):
        m.table_view(t).copy_(quantize_rowwise_nbit(torch.randn(r, d), b).to(device))
    # bags long enough that the id fetch (32 per round) and the row unrolling both wrap around
    g = torch.Generator().manual_seed(0)
    B = 17
    lens = torch.randint(0, 80, (3 * B,), generator=g)
    rows = [300, 50, 50]
    vals = torch.cat([torch.randint(0, rows[k], (int(lens[k * B:(k + 1) * B].sum()),), generator=g) for k in range(3)])
    off = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)])
    want = m(vals.to(device), off.to(device))
    out = torch.full((B + 2, 400), -1.0, device=device)
    cols = [132, 0, 260]  # any order, with gaps; multiples of 4 (the kernel stores four elements at a time)
    m.forward_into(vals.to(device), off.to(device), None, out, cols)
    for f, c in enumerate(cols):
        d = m.D_offsets[f + 1] - m.D_offsets[f]
        torch.testing.assert_close(out[:B, c: c + d], want[:, m.D_offsets[f]: m.D_offsets[f + 1]], rtol=1e-5, atol=1e-5)
    with pytest.raises(ValueError):
        m.forward_into(vals.to(device), off.to(device), None, out, [130, 0, 260])
    assert bool((out[B:] == -1).all()) and bool((out[:, 128:132] == -1).all()) and bool((out[:, 196:260] == -1).all())


def test_qtbe_forward_into_cpu():
    _forward_into_case("cpu")


@pytest.mark.gpu
def test_qtbe_forward_into_gpu():
    _forward_into_case("cuda")


@pytest.mark.gpu
@pytest.mark.parametrize("bits,D", [(8, 128), (8, 32), (8, 256), (4, 128), (4, 32), (4, 256)])
@pytest.mark.parametrize("pooling", [0, 1, 2])
def test_qtbe_shared_lane_kernel_matches_cpu(bits, D, pooling):
    """Tables that all share one low-bit row format take the kernel that spreads a warp's lanes over several rows per load:
    bags longer than one round of ids, weighted, mean and unpooled forms against the host implementation."""
    from torchrec_b200.modules.embedding_configs import PoolingMode
    from torchrec_b200.ops.qtbe import QuantTableBatchedEmbeddingBags
    from torchrec_b200.ops.quant_ops import quantize_rowwise_nbit

    torch.manual_seed(bits * D + pooling)
    specs = [(300, D, bits), (50, D, bits)]
    ftm = [0, 1, 1]
    cpu = QuantTableBatchedEmbeddingBags(specs, ftm, PoolingMode(pooling), torch.float32)
    assert cpu._uniform_bits == bits
    for t, (r, d, b) in enumerate(specs):
        cpu.table_view(t).copy_(quantize_rowwise_nbit(torch.randn(r, d), b))
    gpu = QuantTableBatchedEmbeddingBags(specs, ftm, PoolingMode(pooling), torch.float32, device="cuda")
    gpu.weights.copy_(cpu.weights)
    g = torch.Generator().manual_seed(1)
    B = 19
    lens = torch.randint(0, 90, (3 * B,), generator=g)
    lens[5] = 0
    rows = [300, 50, 50]
    vals = torch.cat([torch.randint(0, rows[k], (int(lens[k * B:(k + 1) * B].sum()),), generator=g) for k in range(3)])
    off = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)])
    psw = torch.rand(vals.numel(), generator=g) if pooling == 0 else None
    ref = cpu(vals, off, psw)
    out = gpu(vals.cuda(), off.cuda(), None if psw is None else psw.cuda())
    gpu.check_error()
    torch.testing.assert_close(out.cpu(), ref, rtol=1e-4, atol=1e-3)
