"""quantize -> shard -> serve on CPU "devices" (cf. ``torchrec/inference/tests/test_inference.py``)."""
import torch

from torchrec_b200.models.dlrm import DLRM
from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


def _model():
    torch.manual_seed(0)
    tables = [EmbeddingBagConfig(name=f"t{i}", num_embeddings=50 + 10 * i, embedding_dim=16, feature_names=[f"f{i}"]) for i in range(4)]
    return DLRM(EmbeddingBagCollection(tables), dense_in_features=8, dense_arch_layer_sizes=[16, 16], over_arch_layer_sizes=[8, 1]).eval()


def _batch(B=7):
    g = torch.Generator().manual_seed(1)
    lens = torch.randint(1, 4, (4 * B,), generator=g)
    vals = torch.cat([torch.randint(0, 50 + 10 * i, (int(lens[i * B:(i + 1) * B].sum()),), generator=g) for i in range(4)])
    return torch.randn(B, 8, generator=g), KeyedJaggedTensor.from_lengths_sync(keys=[f"f{i}" for i in range(4)], values=vals, lengths=lens)


def test_quantize_shard_and_predict():
    from torchrec_b200.distributed.quant_embeddingbag import ShardedQuantEmbeddingBagCollection
    from torchrec_b200.inference.modules import PredictModule, assign_weights_to_tbe, get_table_to_weights_from_tbe, quantize_inference_model, shard_quant_model
    from torchrec_b200.quant.embedding_modules import EmbeddingBagCollection as QEBC

    model = _model()
    dense, kjt = _batch()
    with torch.no_grad():
        ref = model(dense, kjt)
    q = quantize_inference_model(model)
    assert isinstance(q.sparse_arch.embedding_bag_collection, QEBC)
    with torch.no_grad():
        out_q = q(dense, kjt)
    torch.testing.assert_close(out_q, ref, rtol=0, atol=0.05)
    sharded, plan = shard_quant_model(q, world_size=2, compute_device="cpu")
    assert isinstance(sharded.sparse_arch.embedding_bag_collection, ShardedQuantEmbeddingBagCollection)
    ranks = sorted(ps.ranks[0] for ps in plan.plan["sparse_arch.embedding_bag_collection"].values())
    assert ranks == [0, 0, 1, 1]

    class Served(PredictModule):
        def predict_forward(self, batch):
            return {"default": self.predict_module(batch["float_features"], batch["id_list_features"])}

    served = Served(sharded, device="cpu")
    out = served({"float_features": dense, "id_list_features": kjt})["default"]
    torch.testing.assert_close(out, out_q)
    # hot swap: zero tables -> the sparse contribution vanishes and comes back after restoring
    snap = {k: [(w.clone(), None) for w, _ in v] for k, v in get_table_to_weights_from_tbe(sharded).items()}
    assign_weights_to_tbe(sharded, {k: [(torch.zeros_like(w), None) for w, _ in v] for k, v in snap.items()})
    assert not torch.allclose(served({"float_features": dense, "id_list_features": kjt})["default"], out_q)
    assign_weights_to_tbe(sharded, snap)
    torch.testing.assert_close(served({"float_features": dense, "id_list_features": kjt})["default"], out_q)
