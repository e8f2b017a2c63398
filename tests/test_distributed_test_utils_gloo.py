"""The sharding test fixtures themselves: input generation, the small model, and the sharded-vs-unsharded harness."""
import pytest
import torch

from torchrec_b200.test_utils.multi_process import run_multi_process


def _tables():
    from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig

    tables = [EmbeddingBagConfig(name=f"table_{i}", embedding_dim=8 + 8 * (i % 2), num_embeddings=40 + 10 * i, feature_names=[f"feature_{i}"]) for i in range(4)]
    weighted = [EmbeddingBagConfig(name=f"weighted_table_{i}", embedding_dim=8, num_embeddings=30 + 10 * i, feature_names=[f"weighted_feature_{i}"]) for i in range(2)]
    return tables, weighted


def test_model_input_generate_splits_global_batch():
    from torchrec_b200.distributed.test_utils.test_model import ModelInput, TestSparseNN

    tables, weighted = _tables()
    whole, parts = ModelInput.generate(batch_size=3, world_size=2, num_float_features=5, tables=tables, weighted_tables=weighted, pooling_avg=2, random_seed=7)
    assert whole.float_features.shape == (6, 5) and len(parts) == 2 and parts[1].float_features.shape == (3, 5)
    assert torch.equal(torch.cat([p.label for p in parts]), whole.label)
    for key in whole.idlist_features.keys():
        g = whole.idlist_features[key]
        assert torch.equal(torch.cat([p.idlist_features[key].lengths() for p in parts]), g.lengths())
        assert torch.equal(torch.cat([p.idlist_features[key].values() for p in parts]), g.values())
    gw = whole.idscore_features["weighted_feature_1"]
    assert torch.equal(torch.cat([p.idscore_features["weighted_feature_1"].weights() for p in parts]), gw.weights())
    again, _ = ModelInput.generate(batch_size=3, world_size=2, num_float_features=5, tables=tables, weighted_tables=weighted, pooling_avg=2, random_seed=7)
    assert torch.equal(again.idlist_features.values(), whole.idlist_features.values())

    model = TestSparseNN(tables=tables, num_float_features=5, weighted_tables=weighted)
    loss, pred = model(whole)
    assert pred.shape == (6,) and loss.dim() == 0
    loss.backward()
    model.eval()
    assert model(parts[0]).shape == (3,)


def _rank(rank, world_size, sharding_type):
    from torchrec_b200.distributed.embedding_types import EmbeddingComputeKernel
    from torchrec_b200.distributed.test_utils.test_sharding import create_test_sharder, sharding_single_rank_test

    tables, weighted = _tables()
    sharders = [create_test_sharder("embedding_bag_collection", sharding_type, EmbeddingComputeKernel.FUSED.value, fused_params={"learning_rate": 0.1, "optimizer": "exact_sgd"})]
    sharding_single_rank_test(rank, world_size, tables=tables, weighted_tables=weighted, sharders=sharders, backend="gloo")


@pytest.mark.parametrize("sharding_type", ["table_wise", "row_wise"])
def test_sharding_single_rank_harness(sharding_type):
    run_multi_process(_rank, world_size=2, sharding_type=sharding_type)


def test_tables_config_and_td_input():
    from torchrec_b200.distributed.test_utils.test_input import TdModelInput
    from torchrec_b200.distributed.test_utils.test_tables import EmbeddingTablesConfig

    cfg = EmbeddingTablesConfig(num_unweighted_features=3, num_weighted_features=2, embedding_feature_dim=16,
                                additional_tables=[[{"name": "extra", "embedding_dim": 16, "num_embeddings": 77, "feature_names": ["fx"]}], [], [
                                    {"name": "own_group", "embedding_dim": 8, "num_embeddings": 5, "feature_names": ["fo"]}]])
    unweighted, weighted, third = cfg.generate_tables()
    assert [t.name for t in unweighted] == ["table_0", "table_1", "table_2", "extra"] and unweighted[0].num_embeddings == 100_000
    assert [t.feature_names[0] for t in weighted] == ["weighted_feature_0", "weighted_feature_1"] and third[0].embedding_dim == 8

    tables, _ = _tables()
    whole, parts = TdModelInput.generate(batch_size=2, world_size=2, num_float_features=4, tables=tables, weighted_tables=[], pooling_avg=2, random_seed=3)
    assert isinstance(whole.idlist_features, dict) and len(parts) == 2
    kjt = parts[0].to_kjt()
    assert kjt.keys() == [f"feature_{i}" for i in range(4)] and kjt.stride() == 2
