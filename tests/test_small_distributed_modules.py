"""fused_params keys, the width bucketer, inference introspection helpers and the package version."""
import torch
from torch import nn

from torchrec_b200.distributed import fused_params as fp
from torchrec_b200.distributed.embedding_dim_bucketer import EmbDimBucketer, EmbDimBucketerPolicy
from torchrec_b200.distributed.infer_utils import get_all_torchrec_modules, get_non_scriptable_trec_module, get_path_device_tuples
from torchrec_b200.modules.embedding_configs import DataType, EmbeddingBagConfig
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection


def test_version():
    import torchrec_b200.version as v

    assert v.__version__.count(".") == 2


def test_fused_params_helpers():
    params = {fp.FUSED_PARAM_REGISTER_TBE_BOOL: True, fp.FUSED_PARAM_TBE_ROW_ALIGNMENT: 16, fp.FUSED_PARAM_LENGTHS_TO_OFFSETS_LOOKUP: True,
              fp.FUSED_PARAM_SSD_TABLE_LIST: ["t"], "learning_rate": 0.1, "cache_load_factor": 0.2}
    assert fp.is_fused_param_register_tbe(params) and not fp.is_fused_param_register_tbe(None) and not fp.is_fused_param_register_tbe({})
    assert fp.get_fused_param_tbe_row_alignment(params) == 16 and fp.get_fused_param_tbe_row_alignment({}) is None
    assert fp.fused_param_lengths_to_offsets_lookup(params) and not fp.fused_param_lengths_to_offsets_lookup(None)
    assert fp.fused_param_bounds_check_mode(params) is None
    assert not fp.is_fused_param_quant_state_dict_split_scale_bias(params)
    assert fp.tbe_fused_params(params) == {"learning_rate": 0.1, "cache_load_factor": 0.2}
    assert fp.tbe_fused_params(None) is None and fp.tbe_fused_params({}) is None

    class Lookup(nn.Module, fp.TBEToRegisterMixIn):
        def __init__(self):
            super().__init__()
            self.k = nn.Identity()

        def get_tbes_to_register(self):
            return {self.k: "cfg"}

    lk = Lookup()
    assert fp.get_tbes_to_register_from_iterable([nn.Linear(1, 1), lk]) == {lk.k: "cfg"}


class _T:
    def __init__(self, cols, dt=DataType.FP32):
        self.local_cols, self.data_type = cols, dt


def test_dim_bucketer_policies():
    tables = [_T(16), _T(32), _T(48), _T(64), _T(32), _T(64, DataType.FP16), _T(256)]
    one = EmbDimBucketer(tables, EmbDimBucketerPolicy.SINGLE_BUCKET)
    assert one.bucket_count() == 1 and one.get_bucket(256, DataType.FP32) == 0
    every = EmbDimBucketer(tables, EmbDimBucketerPolicy.ALL_BUCKETS)
    # byte widths: 64, 128, 192, 256, 128, 128, 1024 -> 5 distinct
    assert every.bucket_count() == 5
    assert every.get_bucket(32, DataType.FP32) == every.get_bucket(64, DataType.FP16)
    line = EmbDimBucketer(tables, EmbDimBucketerPolicy.CACHELINE_BUCKETS)
    # 128-byte line counts: 0, 1, 1, 2, 1, 1, 8 -> 4 groups
    assert line.bucket_count() == 4
    assert line.get_bucket(32, DataType.FP32) == line.get_bucket(48, DataType.FP32) != line.get_bucket(64, DataType.FP32)


def test_infer_utils_module_search_and_devices():
    ebc = EmbeddingBagCollection(tables=[EmbeddingBagConfig(name="t", embedding_dim=8, num_embeddings=10, feature_names=["f"])])

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.sparse = nn.Sequential(ebc)
            self.dense = nn.Linear(4, 2)
            self.extra = [torch.zeros(2)]

    net = Net()
    found = get_all_torchrec_modules(net)
    assert list(found) == ["sparse.0"] and found["sparse.0"] is ebc
    assert get_non_scriptable_trec_module(net) == {}
    paths = dict(get_path_device_tuples(net))
    assert paths["dense.weight"] == "cpu" and paths["extra[0]"] == "cpu"
    assert any(p.startswith("sparse.0.embedding_bags.t") for p in paths)


def test_quant_utils_fx_names_and_meta_to_cpu():
    from torchrec_b200.modules.embedding_configs import DataType as DT
    from torchrec_b200.quant.embedding_modules import EmbeddingBagCollection as QEBC
    from torchrec_b200.quant.utils import meta_to_cpu_placement, recursive_populate_fx_names

    tables = [EmbeddingBagConfig(name="a", embedding_dim=8, num_embeddings=10, feature_names=["fa"], data_type=DT.INT8),
              EmbeddingBagConfig(name="b", embedding_dim=8, num_embeddings=10, feature_names=["fb"], data_type=DT.INT8)]

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.q = QEBC(tables, is_weighted=False, device=torch.device("meta"))
            self.keep = QEBC(tables, is_weighted=False, device=torch.device("cpu"))

    net = Net()
    old_q, old_keep = net.q, net.keep
    recursive_populate_fx_names(net)
    assert old_q._emb_modules[0]._fx_path == "emb_module.a,b"
    meta_to_cpu_placement(net)
    assert net.q is not old_q and net.keep is old_keep
    assert net.q.device.type == "cpu" and [c.name for c in net.q.embedding_bag_configs()] == ["a", "b"]


def test_grouped_position_weighted_module():
    from torchrec_b200.distributed.grouped_position_weighted import GroupedPositionWeightedModule
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    m = GroupedPositionWeightedModule({"a": 3, "c": 2})
    with torch.no_grad():
        m.position_weights["a"].copy_(torch.tensor([1.0, 2.0, 3.0]))
        m.position_weights["c"].copy_(torch.tensor([10.0, 20.0]))
    kjt = KeyedJaggedTensor.from_lengths_sync(keys=["a", "b", "c"], values=torch.arange(10), lengths=torch.tensor([3, 1, 2, 0, 1, 3]))
    out = m(kjt)
    # a: bags [0,1,2],[0]; b: [0,1],[]; c: [0],[0,1,2 -> clamped to 1]
    torch.testing.assert_close(out.weights(), torch.tensor([1.0, 2.0, 3.0, 1.0, 1.0, 1.0, 10.0, 10.0, 20.0, 20.0]))
    out.weights().sum().backward()
    torch.testing.assert_close(m.position_weights["a"].grad, torch.tensor([2.0, 1.0, 1.0]))
    torch.testing.assert_close(m.position_weights["c"].grad, torch.tensor([2.0, 2.0]))
    assert sorted(m.state_dict()) == ["position_weights.a", "position_weights.c"]
    assert [n for n, _ in m.named_parameters("fp")] == ["fp.position_weights.a", "fp.position_weights.c"]
    # positions carried as weights (as after a row-wise input dist) are used instead of the offsets
    carried = KeyedJaggedTensor.from_lengths_sync(keys=["a"], values=torch.arange(2), lengths=torch.tensor([2]), weights=torch.tensor([2.0, 0.0]))
    torch.testing.assert_close(m(carried).weights(), torch.tensor([3.0, 1.0]))


def test_alias_import_paths():
    from torchrec_b200.distributed.batched_embedding_kernel import TableBatchedEmbeddingSlice as A
    from torchrec_b200.distributed.composable.table_batched_embedding_slice import TableBatchedEmbeddingSlice as B
    from torchrec_b200.distributed.embedding_kernel import BaseEmbedding, get_state_dict  # noqa: F401

    assert A is B


def test_sharded_tbes_weights_spec():
    from torchrec_b200.distributed.quant_embeddingbag import ShardedQuantEmbeddingBagCollection
    from torchrec_b200.distributed.quant_state import WeightSpec, get_param_id_from_type, sharded_tbes_weights_spec
    from torchrec_b200.distributed.types import ParameterSharding, ShardingEnv
    from torchrec_b200.modules.embedding_configs import DataType as DT
    from torchrec_b200.quant.embedding_modules import EmbeddingBagCollection as QEBC

    tables = [EmbeddingBagConfig(name="a", embedding_dim=8, num_embeddings=10, feature_names=["fa"], data_type=DT.INT8),
              EmbeddingBagConfig(name="b", embedding_dim=16, num_embeddings=20, feature_names=["fb"], data_type=DT.INT4)]
    q = QEBC(tables, is_weighted=False, device=torch.device("cpu"))
    sharding = {"a": ParameterSharding(sharding_type="table_wise", compute_kernel="quant", ranks=[0]),
                "b": ParameterSharding(sharding_type="table_wise", compute_kernel="quant", ranks=[1])}
    sharded = ShardedQuantEmbeddingBagCollection(q, sharding, ShardingEnv.from_local(world_size=2, rank=0), device=torch.device("cpu"))
    net = nn.Sequential(sharded)
    spec = sharded_tbes_weights_spec(net)
    assert spec["0.tbes.0.0.a.weight"] == WeightSpec("0.embedding_bags.a.weight", [0, 0], [10, 8], "table_wise")
    assert spec["0.tbes.1.0.b.weight"].shard_sizes == [20, 8]
    assert spec["0.tbes.1.0.b.weight_qscale"].fqn == "0.embedding_bags.b.weight_qscale" and spec["0.tbes.1.0.b.weight_qbias"].shard_sizes == [20, 2]
    assert len(spec) == 6
    assert get_param_id_from_type(True, False, False) == "embedding_bags" and get_param_id_from_type(False, False, False) == "embeddings"


def test_infer_pool_sharding_single_process():
    from torchrec_b200.distributed.sharding.rw_tensor_pool_sharding import InferRwTensorPoolSharding
    from torchrec_b200.distributed.types import ShardingEnv

    sharding = InferRwTensorPoolSharding(pool_size=10, env=ShardingEnv.from_local(world_size=3, rank=0), device=torch.device("cpu"))
    assert sharding.local_pool_size_per_rank == [4, 4, 2]
    pool = torch.arange(10.0).unsqueeze(1).repeat(1, 2)
    shards = [pool[0:4], pool[4:8], pool[8:10]]
    ids_dist = sharding.create_lookup_ids_dist()
    ids = torch.tensor([9, 0, 5, 4, 3, 8])
    parts = ids_dist(ids)
    assert [p.tolist() for p in parts] == [[0, 3], [1, 0], [1, 0]]
    out = sharding.create_lookup_values_dist()([s.index_select(0, p) for s, p in zip(shards, parts)], ids_dist.unbucketize_permute)
    assert torch.equal(out, pool.index_select(0, ids))
