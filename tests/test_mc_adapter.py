"""Managed-collision adapters: construct from table configs, look up raw ids from a huge id space."""
import pytest
import torch

from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig, EmbeddingConfig
from torchrec_b200.modules.mc_adapter import McEmbeddingBagCollectionAdapter, McEmbeddingCollectionAdapter
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


def _materialize(m):
    m.to_empty(device="cpu") if any(p.is_meta for p in m.parameters()) else None
    for p in m.parameters():
        torch.nn.init.normal_(p)


def _kjt():
    return KeyedJaggedTensor.from_lengths_sync(keys=["f1", "f2"], values=torch.tensor([10 ** 12 + 7, 5, 10 ** 15, 5, 99, 123456789]),
                                               lengths=torch.tensor([2, 1, 1, 2]))


@pytest.mark.parametrize("method", ["sort_zch", "mpzch"])
def test_ec_adapter(method):
    tables = [EmbeddingConfig(name="t1", embedding_dim=8, num_embeddings=64, feature_names=["f1"]),
              EmbeddingConfig(name="t2", embedding_dim=8, num_embeddings=64, feature_names=["f2"])]
    ad = McEmbeddingCollectionAdapter(tables, input_hash_size=2 ** 62, device=torch.device("cpu"), world_size=1, zch_method=method, mpzch_num_buckets=4, mpzch_max_probe=16)
    _materialize(ad.mc_embedding_collection._embedding_module)
    out = ad(_kjt())
    assert set(out) == {"f1", "f2"} and out["f1"].values().shape == (3, 8) and out["f2"].values().shape == (3, 8)
    assert len(list(ad.parameters())) == 2 and [c.name for c in ad.embedding_bag_configs()] == ["t1", "t2"]
    out["f1"].values().sum().backward()


def test_ebc_adapter_and_unknown_method():
    tables = [EmbeddingBagConfig(name="t1", embedding_dim=8, num_embeddings=64, feature_names=["f1"]),
              EmbeddingBagConfig(name="t2", embedding_dim=4, num_embeddings=32, feature_names=["f2"])]
    ad = McEmbeddingBagCollectionAdapter(tables, input_hash_size=2 ** 62, device=torch.device("cpu"), world_size=1, zch_method="sort_zch")
    _materialize(ad.mc_embedding_bag_collection._embedding_module)
    kt = ad(_kjt())
    assert kt.values().shape == (2, 12) and kt.keys() == ["f1", "f2"]
    with pytest.raises(NotImplementedError):
        McEmbeddingBagCollectionAdapter(tables, 2 ** 62, torch.device("cpu"), 1, zch_method="")
