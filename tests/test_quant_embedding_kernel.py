"""Shard-level quantized kernels built from a grouped config and from a float kernel."""
import torch

from torchrec_b200.distributed.embedding_types import EmbeddingComputeKernel, GroupedEmbeddingConfig, ShardedEmbeddingTable
from torchrec_b200.distributed.fused_params import get_tbes_to_register_from_iterable
from torchrec_b200.distributed.quant_embedding_kernel import QuantBatchedEmbedding, QuantBatchedEmbeddingBag
from torchrec_b200.modules.embedding_configs import DataType, PoolingType
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class _FloatKernel(torch.nn.Module):
    def __init__(self, config, weights):
        super().__init__()
        self.config, self._w = config, weights

    def split_embedding_weights(self):
        return self._w


def _config(pooling=PoolingType.SUM):
    tables = [ShardedEmbeddingTable(name="a", embedding_dim=16, num_embeddings=40, feature_names=["fa"], local_rows=20, local_cols=16, pooling=pooling, data_type=DataType.FP32),
              ShardedEmbeddingTable(name="b", embedding_dim=16, num_embeddings=12, feature_names=["fb1", "fb2"], local_rows=12, local_cols=16, pooling=pooling, data_type=DataType.FP32)]
    return GroupedEmbeddingConfig(data_type=DataType.FP32, pooling=pooling, is_weighted=False, has_feature_processor=False,
                                  compute_kernel=EmbeddingComputeKernel.QUANT, embedding_tables=tables)


def _kjt(B=5, seed=0):
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(0, 4, (3 * B,), generator=g)
    per = lens.view(3, B).sum(1).tolist()
    vals = torch.cat([torch.randint(0, hi, (n,), generator=g) for hi, n in zip((20, 12, 12), per)])
    return KeyedJaggedTensor(keys=["fa", "fb1", "fb2"], values=vals, lengths=lens)


def test_pooled_kernel_from_float_matches_dequantized_sum():
    torch.manual_seed(0)
    cfg = _config()
    wa, wb = torch.randn(20, 16), torch.randn(12, 16)
    q = QuantBatchedEmbeddingBag.from_float(_FloatKernel(cfg, [wa, wb]), data_type=DataType.INT8)
    kjt = _kjt()
    out = q(kjt)
    assert out.shape == (5, 48)
    jt = kjt.to_dict()
    for col, (key, w) in enumerate((("fa", wa), ("fb1", wb), ("fb2", wb))):
        seg = torch.repeat_interleave(torch.arange(5), jt[key].lengths())
        want = torch.zeros(5, 16).index_add_(0, seg, w[jt[key].values()])
        torch.testing.assert_close(out[:, col * 16:(col + 1) * 16], want, rtol=0.05, atol=0.06)
    names = [n for n, _ in q.named_buffers("k")]
    assert names == ["k.a.weight", "k.b.weight"] and list(q.named_parameters()) == []
    assert get_tbes_to_register_from_iterable([q]) == {q.emb_module: q.config}


def test_sequence_kernel_rows():
    torch.manual_seed(1)
    cfg = _config(PoolingType.NONE)
    wa, wb = torch.randn(20, 16), torch.randn(12, 16)
    q = QuantBatchedEmbedding.from_float(_FloatKernel(cfg, [wa, wb]), data_type=DataType.INT8)
    kjt = _kjt(seed=3)
    rows = q(kjt)
    jt = kjt.to_dict()
    want = torch.cat([wa[jt["fa"].values()], wb[jt["fb1"].values()], wb[jt["fb2"].values()]])
    assert rows.shape == want.shape
    torch.testing.assert_close(rows, want, rtol=0.05, atol=0.03)
