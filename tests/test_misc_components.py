"""Smaller components: datasets, composable shard API, validators, packed int tensors, fused single-device EBC,
feature processors, regroup, delta store (cf. the matching ``tests`` folders of the reference)."""
import os
import warnings

import numpy as np
import pytest
import torch

from torchrec_b200.test_utils.multi_process import MultiProcessContext, run_multi_process


def test_criteo_binary_pipe_splits_rows_over_ranks(tmp_path):
    from torchrec_b200.datasets.criteo import CAT_FEATURE_COUNT, INT_FEATURE_COUNT, BinaryCriteoUtils, InMemoryBinaryCriteoIterDataPipe

    rng = np.random.default_rng(0)
    paths = {"dense": [], "sparse": [], "labels": []}
    rows = [10, 7]
    for d, n in enumerate(rows):
        tsv = tmp_path / f"day_{d}.tsv"
        with open(tsv, "w") as f:
            for _ in range(n):
                ints = [str(int(x)) for x in rng.integers(0, 100, INT_FEATURE_COUNT)]
                cats = [format(int(x), "x") for x in rng.integers(0, 2 ** 20, CAT_FEATURE_COUNT)]
                f.write("\t".join([str(int(rng.integers(0, 2)))] + ints + cats) + "\n")
        out = {k: str(tmp_path / f"day_{d}_{k}.npy") for k in paths}
        BinaryCriteoUtils.tsv_to_npys(str(tsv), out["dense"], out["sparse"], out["labels"])
        for k in paths:
            paths[k].append(out[k])
    seen = 0
    firsts = []
    for rank in range(2):
        pipe = InMemoryBinaryCriteoIterDataPipe("train", paths["dense"], paths["sparse"], paths["labels"], batch_size=4, rank=rank, world_size=2, hashes=[1000] * CAT_FEATURE_COUNT)
        batches = list(pipe)
        assert len(batches) == len(pipe)
        for b in batches:
            assert b.sparse_features.keys()[0] == "cat_0" and b.sparse_features.values().max() < 1000
            assert b.dense_features.shape[1] == INT_FEATURE_COUNT and b.sparse_features.stride() == b.labels.numel()
            seen += b.labels.numel()
        firsts.append(batches[0].dense_features[0].clone())
    assert seen == sum(rows) and not torch.equal(firsts[0], firsts[1])
    r, _ = BinaryCriteoUtils.get_file_row_ranges_and_remainder(rows, rank=1, world_size=2)
    assert r == {0: (9, 9), 1: (0, 6)}


def test_movielens_rows(tmp_path):
    from torchrec_b200.datasets.movielens import movielens_20m

    (tmp_path / "ratings.csv").write_text("userId,movieId,rating,timestamp\n1,10,4.5,100\n2,11,3.0,101\n")
    (tmp_path / "movies.csv").write_text("movieId,title,genres\n10,Heat,Crime\n11,Ran,Drama\n")
    rows = list(movielens_20m(str(tmp_path), include_movies_data=True))
    assert rows[0] == {"userId": 1, "movieId": 10, "rating": 4.5, "timestamp": 100, "title": "Heat", "genres": "Crime"}


def _shard_api_worker(rank, world_size):
    from torchrec_b200.distributed import sharding_plan as sp
    from torchrec_b200.distributed.embeddingbag import ShardedEmbeddingBagCollection
    from torchrec_b200.distributed.shard import shard, shard_modules
    from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig
    from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    with MultiProcessContext(rank, world_size, "gloo") as ctx:
        torch.manual_seed(0)
        tables = [EmbeddingBagConfig(name=f"t{i}", num_embeddings=20, embedding_dim=8, feature_names=[f"f{i}"]) for i in range(2)]
        ebc = EmbeddingBagCollection(tables)
        ref_w = {n: m.weight.detach().clone() for n, m in ebc.embedding_bags.items()}
        sharded = shard(ebc, {"t0": sp.table_wise(rank=0), "t1": sp.row_wise()}, env=ctx.pg, device=torch.device("cpu"))
        assert isinstance(sharded, ShardedEmbeddingBagCollection)
        model = torch.nn.Sequential(EmbeddingBagCollection(tables))
        model = shard_modules(model, env=ctx.pg, device=torch.device("cpu"))
        assert isinstance(model[0], ShardedEmbeddingBagCollection)
        kjt = KeyedJaggedTensor.from_lengths_sync(keys=["f0", "f1"], values=torch.tensor([1, 2, 3, 4]), lengths=torch.tensor([1, 1, 2, 0]))
        out = model[0](kjt).wait()
        assert out.values().shape == (2, 16)


def test_composable_shard_api_gloo():
    run_multi_process(_shard_api_worker, world_size=2)


def test_kjt_validator_and_packed_ints():
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor
    from torchrec_b200.sparse.jagged_tensor_validator import validate_keyed_jagged_tensor
    from torchrec_b200.types import UInt2Tensor, UInt4Tensor

    validate_keyed_jagged_tensor(KeyedJaggedTensor.from_lengths_sync(keys=["a", "b"], values=torch.arange(5), lengths=torch.tensor([2, 1, 0, 2])))
    with pytest.raises(ValueError, match="unique"):
        validate_keyed_jagged_tensor(KeyedJaggedTensor(keys=["a", "a"], values=torch.arange(2), lengths=torch.tensor([1, 1])))
    with pytest.raises(ValueError, match="Sum of lengths"):
        validate_keyed_jagged_tensor(KeyedJaggedTensor(keys=["a"], values=torch.arange(3), lengths=torch.tensor([1, 1])))
    v = torch.randint(0, 16, (3, 8))
    assert torch.equal(UInt4Tensor.pack(v).unpack(), v.to(torch.uint8)) and UInt4Tensor.pack(v).shape == (3, 8)
    v2 = torch.randint(0, 4, (2, 8))
    assert torch.equal(UInt2Tensor.pack(v2).unpack(), v2.to(torch.uint8))


def test_fused_ebc_updates_like_plain_sgd():
    import copy

    from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig, PoolingType
    from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
    from torchrec_b200.modules.fused_embedding_modules import FusedEmbeddingBagCollection, fuse_embedding_optimizer
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    torch.manual_seed(0)
    tables = [EmbeddingBagConfig(name="t0", num_embeddings=20, embedding_dim=8, feature_names=["f0"]),
              EmbeddingBagConfig(name="t1", num_embeddings=10, embedding_dim=4, feature_names=["f1"], pooling=PoolingType.MEAN)]
    ebc = EmbeddingBagCollection(tables)
    ref = copy.deepcopy(ebc)
    f = fuse_embedding_optimizer(torch.nn.Sequential(ebc), torch.optim.SGD, {"lr": 0.5}, torch.device("cpu"))[0]
    assert isinstance(f, FusedEmbeddingBagCollection)
    kjt = KeyedJaggedTensor.from_lengths_sync(keys=["f0", "f1"], values=torch.tensor([1, 2, 3, 4, 5, 6]), lengths=torch.tensor([2, 1, 1, 2]))
    o, r = f(kjt), ref(kjt)
    torch.testing.assert_close(o.values(), r.values())
    o.values().sum().backward(); r.values().sum().backward()
    torch.optim.SGD(ref.parameters(), lr=0.5).step()
    for n in ("t0", "t1"):
        torch.testing.assert_close(f.embedding_bags[n].weight.detach(), ref.embedding_bags[n].weight.detach())
    assert sorted(f.fused_optimizer.params.keys()) == ["embedding_bags.t0.weight", "embedding_bags.t1.weight"]


def test_position_weighted_fp_ebc_and_regroup():
    from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig
    from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
    from torchrec_b200.modules.feature_processor_ import PositionWeightedModule, PositionWeightedModuleCollection
    from torchrec_b200.modules.fp_embedding_modules import FeatureProcessedEmbeddingBagCollection
    from torchrec_b200.modules.regroup import KTRegroupAsDict
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor, KeyedTensor

    kjt = KeyedJaggedTensor.from_lengths_sync(keys=["f0", "f1"], values=torch.tensor([1, 2, 3, 4, 5, 6]), lengths=torch.tensor([2, 1, 0, 3]))
    ebc = EmbeddingBagCollection([EmbeddingBagConfig(name="t0", num_embeddings=10, embedding_dim=4, feature_names=["f0", "f1"])], is_weighted=True)
    fpc = PositionWeightedModuleCollection({"f0": 3, "f1": 3})
    with torch.no_grad():
        fpc.position_weights["f1"].copy_(torch.tensor([1.0, 2.0, 3.0]))
    a = FeatureProcessedEmbeddingBagCollection(ebc, fpc)(kjt)
    b = FeatureProcessedEmbeddingBagCollection(ebc, {"f1": PositionWeightedModule(3)})
    with torch.no_grad():
        b._feature_processors["f1"].position_weight.copy_(torch.tensor([1.0, 2.0, 3.0]))
    torch.testing.assert_close(a.values(), b(kjt).values())
    w = ebc.embedding_bags["t0"].weight.detach()
    torch.testing.assert_close(a["f1"][1], w[4] * 1 + w[5] * 2 + w[6] * 3)
    kt1 = KeyedTensor(keys=["a", "b"], length_per_key=[2, 3], values=torch.arange(10.0).view(2, 5))
    kt2 = KeyedTensor(keys=["c"], length_per_key=[1], values=torch.tensor([[9.0], [8.0]]))
    got = KTRegroupAsDict([["c", "a"], ["b"]], ["x", "y"])([kt1, kt2])
    ref = KeyedTensor.regroup_as_dict([kt1, kt2], [["c", "a"], ["b"]], ["x", "y"])
    for k in got:
        torch.testing.assert_close(got[k], ref[k])


def test_delta_store_first_last_and_compaction():
    from torchrec_b200.distributed.model_tracker import DeltaStore, EmbdUpdateMode

    s = DeltaStore(EmbdUpdateMode.FIRST)
    s.append(0, "t", torch.tensor([3, 1, 3]), torch.tensor([[1.0], [2.0], [3.0]]))
    s.append(1, "t", torch.tensor([1, 5]), torch.tensor([[9.0], [8.0]]))
    d = s.get_delta()["t"]
    assert d.ids.tolist() == [1, 3, 5] and d.states.view(-1).tolist() == [2.0, 1.0, 8.0]
    s.compact(0, 2)
    assert len(s.per_fqn_lookups["t"]) == 1
    s.delete(up_to_idx=1)
    assert s.get_delta() == {}
    last = DeltaStore(EmbdUpdateMode.LAST)
    last.append(0, "t", torch.tensor([3, 1, 3]), torch.tensor([[1.0], [2.0], [3.0]]))
    assert last.get_delta()["t"].states.view(-1).tolist() == [2.0, 3.0]


def test_experimental_warns_once():
    from torchrec_b200.utils.experimental import experimental

    @experimental
    def f():
        return 1

    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        f(); f()
    assert len(w) == 1


def test_cmd_conf_builds_flags_from_dataclasses(tmp_path):
    import dataclasses
    import sys

    from torchrec_b200.distributed.benchmark.benchmark_base import cmd_conf

    @dataclasses.dataclass
    class Opt:
        steps: int = 3
        name: str = "a"
        flag: bool = False

    seen = {}

    @cmd_conf
    def main(opt: Opt) -> None:
        seen["opt"] = opt

    cfg = tmp_path / "c.yml"
    cfg.write_text("steps: 7\nname: from_yaml\n")
    old = sys.argv
    try:
        sys.argv = ["prog", "--yaml_config", str(cfg), "--name", "cli"]
        main()
    finally:
        sys.argv = old
    assert seen["opt"].steps == 7 and seen["opt"].name == "cli" and seen["opt"].flag is False


def test_bert4rec_forward_backward():
    from torchrec_b200.models.bert4rec import BERT4Rec
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    torch.manual_seed(0)
    m = BERT4Rec(vocab_size=50, max_len=6, emb_dim=16, nhead=2, num_layers=1, dropout=0.0)
    lengths = torch.tensor([3, 6, 1])
    kjt = KeyedJaggedTensor(keys=["item"], values=torch.randint(0, 50, (10,)), lengths=lengths)
    out = m(kjt)
    assert out.shape == (3, 6, 50)
    out.sum().backward()
    assert m.history.ec.embeddings["item_embedding"].weight.grad is not None
    # padded positions do not influence valid ones: changing nothing but the padding mask input length keeps row 1 identical
    m.eval()
    with torch.no_grad():
        a = m(kjt)[1]
        kjt2 = KeyedJaggedTensor(keys=["item"], values=kjt.values()[3:9], lengths=torch.tensor([6]))
        b = m(kjt2)[0]
    torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-5)
    pos = torch.tensor([0, 7])
    sl = m.sampled_logits(kjt, pos, torch.tensor([4, 5]), torch.tensor([1, 2, 3]))
    assert sl.shape == (2, 4)
    torch.testing.assert_close(sl[:, 0], m(kjt).reshape(-1, 50)[pos, torch.tensor([4, 5])], rtol=1e-4, atol=1e-5)
