"""DeepFM and transformer-interaction DLRM: shapes, gradients and a hand-computed forward."""
import torch

from torchrec_b200.models.deepfm import FMInteractionArch, SimpleDeepFMNN, SimpleDeepFMNNWrapper
from torchrec_b200.models.experimental.transformerdlrm import DLRM_Transformer, InteractionTransformerArch
from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor, KeyedTensor


def _ebc(D=8):
    return EmbeddingBagCollection(tables=[
        EmbeddingBagConfig(name="t1", embedding_dim=D, num_embeddings=50, feature_names=["f1", "f3"]),
        EmbeddingBagConfig(name="t2", embedding_dim=D, num_embeddings=30, feature_names=["f2"]),
    ])


def _kjt(B=4):
    lengths = torch.tensor([2, 0, 1, 1, 1, 3, 0, 2, 1, 1, 1, 1])
    return KeyedJaggedTensor.from_lengths_sync(keys=["f1", "f3", "f2"], values=torch.randint(0, 30, (int(lengths.sum()),)), lengths=lengths)


def test_fm_interaction_matches_hand_computation():
    torch.manual_seed(0)
    B, D, DI = 4, 8, 5
    arch = FMInteractionArch(fm_in_features=3 * D, sparse_feature_names=["a", "b"], deep_fm_dimension=DI)
    dense = torch.randn(B, D)
    sp = torch.randn(B, 2 * D)
    out = arch(dense, KeyedTensor(keys=["a", "b"], length_per_key=[D, D], values=sp))
    x = torch.cat([dense, sp], dim=1)
    deep = torch.relu(arch.deep_fm.dense_module[0](x))
    fm = 0.5 * (x.sum(1, keepdim=True) ** 2 - (x * x).sum(1, keepdim=True))
    torch.testing.assert_close(out, torch.cat([dense, deep, fm], dim=1))
    assert out.shape == (B, D + DI + 1)
    assert torch.equal(FMInteractionArch(D, [], DI)(dense, KeyedTensor(keys=[], length_per_key=[], values=torch.empty(B, 0))), dense)


def test_simple_deepfm_forward_backward():
    torch.manual_seed(1)
    model = SimpleDeepFMNN(num_dense_features=10, embedding_bag_collection=_ebc(), hidden_layer_size=20, deep_fm_dimension=5)
    out = model(torch.rand(4, 10), _kjt())
    assert out.shape == (4, 1) and float(out.min()) >= 0.0 and float(out.max()) <= 1.0
    out.sum().backward()
    assert all(p.grad is not None for p in model.parameters())


def test_deepfm_wrapper_trains():
    torch.manual_seed(2)

    class Batch:
        float_features = torch.rand(4, 10)
        idlist_features = _kjt()
        label = torch.tensor([1.0, 0.0, 1.0, 0.0])

    model = SimpleDeepFMNNWrapper(num_dense_features=10, embedding_bag_collection=_ebc(), hidden_layer_size=20, deep_fm_dimension=5)
    opt = torch.optim.SGD(model.parameters(), lr=0.5)
    first = None
    for _ in range(30):
        opt.zero_grad()
        loss, pred = model(Batch)
        loss.backward()
        opt.step()
        first = float(loss) if first is None else first
    assert float(loss) < first
    model.eval()
    assert model(Batch).shape == (4, 1)


def test_transformer_interaction_and_dlrm():
    torch.manual_seed(3)
    B, D, F = 4, 8, 3
    arch = InteractionTransformerArch(num_sparse_features=F, embedding_dim=D, nhead=2, ntransformer_layers=1)
    assert arch(torch.randn(B, D), torch.randn(B, F, D)).shape == (B, (F + 1) * D)
    assert InteractionTransformerArch(0, D, 2, 1)(torch.ones(B, D), torch.empty(B, 0, D)).shape == (B, D)
    model = DLRM_Transformer(_ebc(D), dense_in_features=10, dense_arch_layer_sizes=[16, D], over_arch_layer_sizes=[16, 1], nhead=2, ntransformer_layers=2)
    logits = model(torch.rand(B, 10), _kjt())
    assert logits.shape == (B, 1)
    logits.sum().backward()
    assert model.inter_arch.interarch_TE.layers[0].linear1.weight.grad is not None
