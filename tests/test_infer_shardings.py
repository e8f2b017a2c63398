"""Inference sharding strategies on two virtual devices (host): request -> input distribution -> all-device quantized lookup ->
output distribution, against plain torch on the dequantized tables."""
import pytest
import torch

from torchrec_b200.distributed import sharding_plan as sp
from torchrec_b200.distributed.embedding_sharding import EmbeddingShardingInfo
from torchrec_b200.distributed.quant_embeddingbag import QuantEmbeddingBagCollectionSharder
from torchrec_b200.distributed.types import ShardingEnv
from torchrec_b200.modules.embedding_configs import DataType, EmbeddingTableConfig, PoolingType
from torchrec_b200.ops.quant_ops import dequantize_rowwise_nbit, quantize_rowwise_nbit
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

W = 2
TABLES = [("t0", "f0", 40, 16), ("t1", "f1", 30, 16), ("t2", "f2", 50, 16)]


def _infos(how, pooled):
    sharder = QuantEmbeddingBagCollectionSharder()
    infos = []
    for i, (name, feat, rows, dim) in enumerate(TABLES):
        cfg = EmbeddingTableConfig(name=name, embedding_dim=dim, num_embeddings=rows, feature_names=[feat], data_type=DataType.INT8,
                                   pooling=PoolingType.SUM if pooled else PoolingType.NONE, embedding_names=[feat])
        gen = {"tw": sp.table_wise(rank=i % W), "rw": sp.row_wise(), "cw": sp.column_wise(ranks=[0, 1])}[how]
        ps = gen(torch.empty(rows, dim, device="meta"), W, W, "cpu", sharder)
        infos.append(EmbeddingShardingInfo(embedding_config=cfg, param_sharding=ps, param=torch.empty(rows, dim, device="meta")))
    return infos


def _request(gen, B=6):
    keys = [f for _, f, _, _ in TABLES]
    lengths = torch.randint(0, 4, (len(keys) * B,), generator=gen)
    values = torch.cat([torch.randint(0, rows, (int(lengths[i * B:(i + 1) * B].sum()),), generator=gen) for i, (_, _, rows, _) in enumerate(TABLES)])
    return KeyedJaggedTensor.from_lengths_sync(keys=keys, values=values, lengths=lengths)


def _fill(lookup, gen):
    """Random quantized rows in every shard; returns the dequantized full tables, assembled from the shards' metadata."""
    full = {name: torch.zeros(rows, dim) for name, _, rows, dim in TABLES}
    for per_device in lookup._embedding_lookups_per_rank:
        for kernel in per_device._emb_modules:
            for table, buf in zip(kernel.config.embedding_tables, kernel.split_embedding_weights()):
                w = torch.randn(table.local_rows, table.local_cols, generator=gen)
                buf.copy_(quantize_rowwise_nbit(w, 8))
                r0, c0 = table.local_metadata.shard_offsets
                full[table.name][r0:r0 + table.local_rows, c0:c0 + table.local_cols] = dequantize_rowwise_nbit(buf, table.local_cols, 8)
    return full


def _pooled_oracle(kjt, full):
    cols = []
    for (name, feat, _, _) in TABLES:
        jt = kjt[feat]
        off = jt.offsets()
        cols.append(torch.stack([full[name][jt.values()[int(a):int(b)]].sum(0) for a, b in zip(off[:-1], off[1:])]))
    return cols


@pytest.mark.parametrize("how", ["tw", "rw", "cw"])
def test_pooled_inference_strategies(how):
    from torchrec_b200.distributed.sharding import cw_sharding, rw_sharding, tw_sharding

    gen = torch.Generator().manual_seed(0)
    env = ShardingEnv.from_local(world_size=W, rank=0)
    cpu = torch.device("cpu")
    cls = {"tw": tw_sharding.InferTwEmbeddingSharding, "rw": rw_sharding.InferRwPooledEmbeddingSharding, "cw": cw_sharding.InferCwPooledEmbeddingSharding}[how]
    sharding = cls(_infos(how, True), env, cpu, permute_embeddings=True) if how == "cw" else cls(_infos(how, True), env, cpu)
    idist, lookup, odist = sharding.create_input_dist(cpu), sharding.create_lookup(cpu), sharding.create_output_dist(cpu)
    full = _fill(lookup, gen)
    kjt = _request(gen)
    feats = kjt.permute([kjt.keys().index(f) for f in sharding.feature_names()]) if how != "rw" else kjt
    out = odist(lookup(idist(feats)))
    want = dict(zip([t[0] for t in TABLES], _pooled_oracle(kjt, full)))
    names = sharding.embedding_names()
    dims = sharding.embedding_dims()
    assert out.shape == (6, sum(dims))
    col = 0
    for name, d in zip(names, dims):
        table = next(t[0] for t in TABLES if t[1] == name or name.startswith(t[1]))
        torch.testing.assert_close(out[:, col:col + d].float(), want[table][:, :d] if d == 16 else want[table][:, :d], rtol=1e-3, atol=1e-3)
        col += d


@pytest.mark.parametrize("how", ["tw", "rw"])
def test_sequence_inference_strategies(how):
    from torchrec_b200.distributed.sharding import rw_sequence_sharding, tw_sequence_sharding

    gen = torch.Generator().manual_seed(1)
    env = ShardingEnv.from_local(world_size=W, rank=0)
    cpu = torch.device("cpu")
    cls = {"tw": tw_sequence_sharding.InferTwSequenceEmbeddingSharding, "rw": rw_sequence_sharding.InferRwSequenceEmbeddingSharding}[how]
    sharding = cls(_infos(how, False), env, cpu)
    idist, lookup, odist = sharding.create_input_dist(cpu), sharding.create_lookup(cpu), sharding.create_output_dist(cpu)
    full = _fill(lookup, gen)
    kjt = _request(gen)
    if how == "tw":
        feats = kjt.permute([kjt.keys().index(f) for f in sharding.feature_names()])
        dist_out = idist(feats)
        rows = odist(lookup(dist_out))
        for per_device, names, local in zip(rows, sharding.feature_names_per_rank(), dist_out.features):
            want = torch.cat([full[next(t[0] for t in TABLES if t[1] == f)][local[f].values()] for f in names])
            torch.testing.assert_close(per_device.float(), want, rtol=1e-3, atol=1e-3)
    else:
        dist_out = idist(kjt)
        rows = torch.cat(odist(lookup(dist_out)))  # (device, feature, sample) order
        ordered = rows.index_select(0, dist_out.unbucketize_permute_tensor.long())
        want = torch.cat([full[name][kjt[feat].values()] for name, feat, _, _ in TABLES])
        torch.testing.assert_close(ordered.float(), want, rtol=1e-3, atol=1e-3)


def test_strategy_factories_and_device_helpers():
    from torchrec_b200.distributed.quant_embedding import create_infer_embedding_sharding
    from torchrec_b200.distributed.quant_embeddingbag import create_infer_embedding_bag_sharding, get_device_from_parameter_sharding, get_device_from_sharding_infos
    from torchrec_b200.distributed.sharding import infer_shardings as inf

    env = ShardingEnv.from_local(world_size=W, rank=0)
    infos = _infos("rw", True)
    assert get_device_from_parameter_sharding(infos[0].param_sharding) == "cpu" and get_device_from_sharding_infos(infos) == "cpu"
    assert isinstance(create_infer_embedding_bag_sharding("row_wise", infos, env, torch.device("cpu")), inf.InferRwPooledEmbeddingSharding)
    assert isinstance(create_infer_embedding_bag_sharding("column_wise", _infos("cw", True), env, torch.device("cpu")), inf.InferCwPooledEmbeddingSharding)
    assert isinstance(create_infer_embedding_sharding("table_wise", _infos("tw", False), env, torch.device("cpu")), inf.InferTwSequenceEmbeddingSharding)
    with pytest.raises(ValueError):
        create_infer_embedding_bag_sharding("grid_shard", infos, env)


def test_inference_bucketize_reports_the_bucket_of_every_id_and_vbe_padding():
    import torch

    from torchrec_b200.distributed.embedding import pad_vbe_kjt_lengths
    from torchrec_b200.distributed.embedding_sharding import bucketize_kjt_inference
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    kjt = KeyedJaggedTensor(keys=["a", "b"], values=torch.tensor([3, 12, 7, 25, 0, 19, 31, 8]), lengths=torch.tensor([2, 1, 3, 2]))
    block = torch.tensor([10, 16])  # feature a: 3 buckets of 10 rows; feature b: of 16 rows (the last one partly used)
    out, permute, mapping = bucketize_kjt_inference(kjt, 3, block, is_sequence=True)
    want = [0, 1, 0, 1, 0, 1, 1, 0]  # a: 3 -> 0, 12 -> 1, 7 -> 0;  b: 25 -> 1, 0 -> 0, 19 -> 1, 31 -> 1, 8 -> 0
    assert mapping.tolist() == want
    assert out.keys() == ["a", "b"] * 3 and int(out.lengths().sum()) == 8
    # the permutation restores the request order from the bucketized one
    local = out.values()[permute]
    assert local.tolist() == [3, 2, 7, 9, 0, 3, 15, 8]
    plain, none_p, none_m = bucketize_kjt_inference(kjt, 3, block)
    assert none_p is None and none_m is None and torch.equal(plain.lengths(), out.lengths())

    vb = KeyedJaggedTensor(keys=["a", "b"], values=torch.arange(6), lengths=torch.tensor([1, 2, 3]), stride_per_key_per_rank=[[1], [2]])
    fixed = pad_vbe_kjt_lengths(vb)
    assert fixed.stride() == 2 and fixed.lengths().tolist() == [1, 0, 2, 3] and torch.equal(fixed.values(), vb.values())
    assert fixed.to_dict()["b"].values().tolist() == [1, 2, 3, 4, 5]
