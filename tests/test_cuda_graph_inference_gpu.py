"""CUDA-graph replay of a quantized DLRM forward equals the eager forward, for requests with different ids and id counts."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_graph_replay_matches_eager():
    from torchrec_b200.inference.cuda_graph import CudaGraphDenseSparseModule
    from torchrec_b200.models.dlrm import DLRM_DCN
    from torchrec_b200.modules.embedding_configs import DataType, EmbeddingBagConfig
    from torchrec_b200.ops import dense_ops
    from torchrec_b200.quant.embedding_modules import EmbeddingBagCollection as QEBC
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    dev = torch.device("cuda:0")
    dense_ops.set_dense_compute_dtype(torch.bfloat16)
    torch.manual_seed(0)
    keys = [f"f{i}" for i in range(6)]
    tables = [EmbeddingBagConfig(name=f"t{i}", embedding_dim=128, num_embeddings=500 + 50 * i, feature_names=[k], data_type=DataType.INT4 if i % 2 else DataType.INT8)
              for i, k in enumerate(keys)]
    q = QEBC(tables=tables, is_weighted=False, device=dev, output_dtype=torch.bfloat16)
    for m in q.embedding_bags.values():
        m.weight.random_(0, 256)
        m.weight[:, -4:] = torch.tensor([1.0 / 64, -1.0], dtype=torch.float16).view(torch.uint8).to(dev)
    model = DLRM_DCN(q, 13, [256, 128], [256, 128, 1], dcn_num_layers=2, dcn_low_rank_dim=64, dense_device=dev).eval()
    B = 256
    g = torch.Generator().manual_seed(1)

    def request(max_len):
        lengths = torch.randint(0, max_len + 1, (len(keys) * B,), generator=g)
        values = torch.cat([torch.randint(0, 500, (int(lengths[i * B:(i + 1) * B].sum()),), generator=g) for i in range(len(keys))])
        return torch.rand(B, 13, generator=g).to(dev), KeyedJaggedTensor(keys=keys, values=values.to(dev), lengths=lengths.to(dev), stride=B)

    d0, k0 = request(6)
    graphed = CudaGraphDenseSparseModule(model, d0, k0, values_capacity=int(k0.values().numel() * 2))
    assert graphed.captured, graphed.capture_error
    for max_len in (6, 2, 9, 0):
        d, k = request(max_len)
        with torch.no_grad():
            want = model(d, k).float()
        got = graphed(d, k).float().clone()
        torch.testing.assert_close(got, want, rtol=2e-2, atol=2e-2)
    assert graphed.replays == 4 and graphed.fallbacks == 0
    d, k = request(40)  # more ids than the static buffer holds: eager fallback
    with torch.no_grad():
        want = model(d, k).float()
    torch.testing.assert_close(graphed(d, k).float(), want, rtol=2e-2, atol=2e-2)
    assert graphed.fallbacks == 1
    for emb in q._emb_modules:
        emb.check_error()
