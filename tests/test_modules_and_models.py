"""Unsharded modules and models against hand-written formulas (cf. ``torchrec/modules/tests``, ``torchrec/models/tests``)."""
import pytest
import torch
from torch import nn

from torchrec_b200.datasets.utils import Batch
from torchrec_b200.models.dlrm import DLRM, DLRM_DCN, DLRM_Projection, DLRMTrain, DenseArch, InteractionArch, OverArch, SparseArch
from torchrec_b200.modules.crossnet import CrossNet, LowRankCrossNet, LowRankMixtureCrossNet, VectorCrossNet
from torchrec_b200.modules.deepfm import DeepFM, FactorizationMachine
from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig, EmbeddingConfig, PoolingType
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection, EmbeddingCollection
from torchrec_b200.modules.mlp import MLP, Perceptron
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


def _kjt():
    return KeyedJaggedTensor(keys=["f1", "f2", "f3"], values=torch.tensor([0, 1, 2, 3, 1, 1, 4, 0, 2]), lengths=torch.tensor([2, 0, 1, 1, 2, 1, 1, 1, 0]))


# ---- embedding collections ---------------------------------------------------------------------------------
@pytest.mark.parametrize("pooling", [PoolingType.SUM, PoolingType.MEAN])
def test_ebc_matches_manual_pooling(pooling):
    torch.manual_seed(0)
    t1 = EmbeddingBagConfig(name="t1", embedding_dim=4, num_embeddings=5, feature_names=["f1", "f3"], pooling=pooling)
    t2 = EmbeddingBagConfig(name="t2", embedding_dim=3, num_embeddings=6, feature_names=["f2"], pooling=pooling)
    ebc = EmbeddingBagCollection(tables=[t1, t2])
    kt = ebc(_kjt())
    assert kt.keys() == ["f1", "f3", "f2"] and kt.length_per_key() == [4, 4, 3] and kt.values().shape == (3, 11)
    w1, w2 = ebc.embedding_bags["t1"].weight, ebc.embedding_bags["t2"].weight
    red = (lambda r: r.mean(0)) if pooling == PoolingType.MEAN else (lambda r: r.sum(0))
    torch.testing.assert_close(kt["f1"][0], red(w1[[0, 1]]))
    torch.testing.assert_close(kt["f1"][1], torch.zeros(4))
    torch.testing.assert_close(kt["f2"][1], red(w2[[1, 1]]))
    torch.testing.assert_close(kt["f3"][1], red(w1[[2]]))
    kt.values().sum().backward()
    assert w1.grad is not None and w2.grad is not None
    assert set(ebc.state_dict().keys()) == {"embedding_bags.t1.weight", "embedding_bags.t2.weight"}


def test_ebc_weighted_and_shared_feature_names():
    t1 = EmbeddingBagConfig(name="t1", embedding_dim=2, num_embeddings=5, feature_names=["f1"])
    t2 = EmbeddingBagConfig(name="t2", embedding_dim=2, num_embeddings=5, feature_names=["f1"])
    ebc = EmbeddingBagCollection(tables=[t1, t2], is_weighted=True)
    kjt = KeyedJaggedTensor(keys=["f1"], values=torch.tensor([1, 2, 3]), lengths=torch.tensor([2, 1]), weights=torch.tensor([0.5, 2.0, 3.0]))
    kt = ebc(kjt)
    assert kt.keys() == ["f1@t1", "f1@t2"]
    w = ebc.embedding_bags["t1"].weight
    torch.testing.assert_close(kt["f1@t1"][0], 0.5 * w[1] + 2.0 * w[2])
    with pytest.raises(ValueError):
        EmbeddingBagCollection(tables=[t1, EmbeddingBagConfig(name="t1", embedding_dim=2, num_embeddings=3, feature_names=["x"])])


def test_embedding_collection_returns_jagged_rows():
    t1 = EmbeddingConfig(name="t1", embedding_dim=4, num_embeddings=5, feature_names=["f1", "f3"])
    t2 = EmbeddingConfig(name="t2", embedding_dim=4, num_embeddings=6, feature_names=["f2"])
    ec = EmbeddingCollection(tables=[t1, t2], need_indices=True)
    out = ec(_kjt())
    assert set(out) == {"f1", "f2", "f3"} and ec.embedding_dim() == 4
    torch.testing.assert_close(out["f2"].values(), ec.embeddings["t2"].weight[[3, 1, 1, 4]])
    assert out["f2"].lengths().tolist() == [1, 2, 1] and out["f2"].weights().tolist() == [3, 1, 1, 4]
    with pytest.raises(ValueError):
        EmbeddingCollection(tables=[t1, EmbeddingConfig(name="t9", embedding_dim=8, num_embeddings=6, feature_names=["z"])])


# ---- dense blocks --------------------------------------------------------------------------------------------------
def test_perceptron_and_mlp():
    torch.manual_seed(0)
    p = Perceptron(6, 3, bias=True, activation=torch.relu)
    x = torch.randn(4, 6)
    torch.testing.assert_close(p(x), torch.relu(x @ p._linear.weight.t() + p._linear.bias))
    mlp = MLP(6, [8, 4, 2], bias=True, activation="relu")
    assert mlp(x).shape == (4, 2) and len(list(mlp.parameters())) == 6
    sig = MLP(6, [3], activation="sigmoid")
    assert ((sig(x) > 0) & (sig(x) < 1)).all()
    sw = MLP(6, [3, 3], activation="swish_layernorm")
    assert sw(x).shape == (4, 3)
    with pytest.raises((ValueError, AssertionError)):
        MLP(6, [3], activation="nope")


def test_crossnets_follow_their_formulas():
    torch.manual_seed(0)
    B, N = 5, 6
    x0 = torch.randn(B, N)
    full = CrossNet(N, 2)
    x = x0
    for l in range(2):
        x = x0 * (x @ full.kernels[l].t() + full.bias[l].view(1, N)) + x
    torch.testing.assert_close(full(x0), x, rtol=1e-5, atol=1e-5)
    lr = LowRankCrossNet(N, 2, low_rank=3)
    x = x0
    for l in range(2):
        x = x0 * ((x @ lr.V_kernels[l].t()) @ lr.W_kernels[l].t() + lr.bias[l].view(1, N)) + x
    torch.testing.assert_close(lr(x0), x, rtol=1e-4, atol=1e-5)
    vec = VectorCrossNet(N, 2)
    x = x0
    for l in range(2):
        x = x0 * (x @ vec.kernels[l].view(N, 1)) + vec.bias[l].view(1, N) + x
    torch.testing.assert_close(vec(x0), x, rtol=1e-5, atol=1e-5)
    mix = LowRankMixtureCrossNet(N, 2, num_experts=3, low_rank=2)
    out = mix(x0)
    assert out.shape == (B, N) and torch.isfinite(out).all()
    out.sum().backward()
    assert all(p.grad is not None for p in mix.parameters())


def test_deepfm_and_factorization_machine():
    torch.manual_seed(0)
    a, b = torch.randn(4, 2, 3), torch.randn(4, 5)
    fm = FactorizationMachine()([a, b])
    flat = torch.cat([a.flatten(1), b], dim=1)
    expect = 0.5 * (flat.sum(1, keepdim=True) ** 2 - (flat * flat).sum(1, keepdim=True))
    torch.testing.assert_close(fm, expect)
    deep = DeepFM(dense_module=nn.Linear(11, 7))
    assert deep([a, b]).shape == (4, 7)


# ---- DLRM family -----------------------------------------------------------------------------------------------------------
def _ebc(D=8):
    return EmbeddingBagCollection(tables=[EmbeddingBagConfig(name=f"t{i}", embedding_dim=D, num_embeddings=20, feature_names=[f"f{i + 1}"]) for i in range(3)])


def test_dlrm_arches_and_interaction_formula():
    torch.manual_seed(0)
    B, D, F = 3, 8, 3
    sparse = SparseArch(_ebc(D))
    s = sparse(_kjt())
    assert s.shape == (B, F, D) and sparse.sparse_feature_names == ["f1", "f2", "f3"]
    dense = DenseArch(13, [16, D])(torch.randn(B, 13))
    assert dense.shape == (B, D)
    inter = InteractionArch(F)(dense, s)
    assert inter.shape == (B, D + (F + 1) * F // 2)
    cat = torch.cat([dense.unsqueeze(1), s], dim=1)
    z = torch.bmm(cat, cat.transpose(1, 2))
    iu = torch.triu_indices(F + 1, F + 1, offset=1)
    torch.testing.assert_close(inter, torch.cat([dense, z[:, iu[0], iu[1]]], dim=1), rtol=1e-4, atol=1e-5)
    assert OverArch(inter.shape[1], [8, 1])(inter).shape == (B, 1)


def test_dlrm_variants_train_step():
    torch.manual_seed(0)
    B = 3
    dense = torch.randn(B, 13)
    kjt = _kjt()
    labels = torch.tensor([1.0, 0.0, 1.0])
    models = [
        DLRM(_ebc(), 13, [16, 8], [16, 1]),
        DLRM_DCN(_ebc(), 13, [16, 8], [16, 1], dcn_num_layers=2, dcn_low_rank_dim=4),
        DLRM_Projection(_ebc(), 13, [16, 8], [16, 1], interaction_branch1_layer_sizes=[16, 16], interaction_branch2_layer_sizes=[16, 8]),
    ]
    for m in models:
        assert m(dense, kjt).shape == (B, 1)
        train = DLRMTrain(m)
        loss, (l2, logits, lab) = train(Batch(dense_features=dense, sparse_features=kjt, labels=labels))
        torch.testing.assert_close(loss, nn.functional.binary_cross_entropy_with_logits(logits, labels))
        loss.backward()
        assert all(p.grad is not None for p in m.parameters()), type(m).__name__
    with pytest.raises((ValueError, AssertionError)):
        DLRM(_ebc(8), 13, [16, 4], [1])  # the dense arch must end in the embedding dimension
    with pytest.raises((ValueError, AssertionError)):
        DLRM_Projection(_ebc(), 13, [16, 8], [16, 1], interaction_branch1_layer_sizes=[16, 15], interaction_branch2_layer_sizes=[16, 8])
