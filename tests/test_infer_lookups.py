"""Inference grouped lookups (one process, all ranks' quantized kernels): table-wise placement over two virtual ranks on the host,
against dequantized tables looked up with plain torch."""
import torch

from torchrec_b200.distributed.embedding_types import EmbeddingComputeKernel, GroupedEmbeddingConfig, InputDistOutputs, KJTList, ShardedEmbeddingTable
from torchrec_b200.modules.embedding_configs import DataType, PoolingType
from torchrec_b200.ops.quant_ops import dequantize_rowwise_nbit, quantize_rowwise_nbit
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


def _table(name, feature, rows, dim, pooling=PoolingType.SUM):
    return ShardedEmbeddingTable(num_embeddings=rows, embedding_dim=dim, name=name, feature_names=[feature], data_type=DataType.INT8, pooling=pooling,
                                 local_rows=rows, local_cols=dim, compute_kernel=EmbeddingComputeKernel.QUANT, embedding_names=[name + "_" + feature])


def _group(tables, pooling=PoolingType.SUM):
    return GroupedEmbeddingConfig(data_type=DataType.INT8, pooling=pooling, is_weighted=False, has_feature_processor=False,
                                  compute_kernel=EmbeddingComputeKernel.QUANT, embedding_tables=tables)


def _kjt(keys, gen, rows, B=5):
    lengths = torch.randint(0, 4, (len(keys) * B,), generator=gen)
    values = torch.cat([torch.randint(0, r, (int(lengths[i * B:(i + 1) * B].sum()),), generator=gen) for i, r in enumerate(rows)])
    return KeyedJaggedTensor.from_lengths_sync(keys=keys, values=values, lengths=lengths)


def test_pooled_and_sequence_inference_lookups_match_dequantized_tables():
    import torchrec_b200.distributed.embedding_lookup as el

    gen = torch.Generator().manual_seed(0)
    cpu = torch.device("cpu")
    per_rank = [[_group([_table("t0", "f0", 50, 16), _table("t1", "f1", 30, 8)])], [], [_group([_table("t2", "f2", 40, 16)])]]
    pooled = el.InferGroupedPooledEmbeddingsLookup(per_rank, world_size=3, device=cpu)
    assert pooled._is_empty_rank == [False, True, False] and len(pooled.get_tbes_to_register()) == 2
    floats = {}
    for name, buf in pooled.named_buffers():
        table = name.split(".")[0]
        dim = {"t0": 16, "t1": 8, "t2": 16}[table]
        w = torch.randn(buf.shape[0], dim, generator=gen)
        buf.copy_(quantize_rowwise_nbit(w, 8))
        floats[table] = dequantize_rowwise_nbit(buf, dim, 8)
    feats = [_kjt(["f0", "f1"], gen, [50, 30]), KeyedJaggedTensor.empty(), _kjt(["f2"], gen, [40])]
    outs = pooled(InputDistOutputs(features=KJTList(feats)))
    assert len(outs) == 2 and outs[0].shape == (5, 24) and outs[1].shape == (5, 16)
    for out, kjt, names in ((outs[0], feats[0], ["t0", "t1"]), (outs[1], feats[2], ["t2"])):
        col = 0
        for key, table in zip(kjt.keys(), names):
            jt = kjt[key]
            w = floats[table]
            want = torch.stack([w[jt.values()[int(lo):int(hi)]].sum(0) for lo, hi in zip(jt.offsets()[:-1], jt.offsets()[1:])])
            torch.testing.assert_close(out[:, col:col + w.shape[1]].float(), want, rtol=1e-3, atol=1e-3)
            col += w.shape[1]
    # state round trip under <table>.weight
    sd = pooled.state_dict()
    assert sorted(sd) == ["t0.weight", "t1.weight", "t2.weight"]
    again = el.InferGroupedPooledEmbeddingsLookup(per_rank, world_size=3, device=cpu)
    for lookup in again._embedding_lookups_per_rank:
        lookup.load_state_dict({k: v for k, v in sd.items() if k in dict(lookup.named_buffers())})
    torch.testing.assert_close(again(InputDistOutputs(features=KJTList(feats)))[0], outs[0])

    seq = el.InferCPUGroupedEmbeddingsLookup([[_group([_table("t0", "f0", 50, 16, PoolingType.NONE)], PoolingType.NONE)]], world_size=1)
    (name, buf), = list(seq.named_buffers())
    buf.copy_(quantize_rowwise_nbit(torch.randn(50, 16, generator=gen), 8))
    kjt = _kjt(["f0"], gen, [50])
    rows = seq(InputDistOutputs(features=KJTList([kjt])))[0]
    torch.testing.assert_close(rows.float(), dequantize_rowwise_nbit(buf, 16, 8)[kjt.values()], rtol=1e-3, atol=1e-3)
