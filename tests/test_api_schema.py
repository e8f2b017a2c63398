"""Public signatures stay call-compatible with the reference package: for each entry, the listed parameter names must exist, in this
order, and the ones the reference gives a default must be optional here too (``torchrec/schema/api_tests/*``)."""
import inspect

import pytest


def _cases():
    from torchrec_b200.distributed.model_parallel import DistributedModelParallel
    from torchrec_b200.distributed.planner import EmbeddingShardingPlanner
    from torchrec_b200.distributed.planner.enumerators import EmbeddingEnumerator
    from torchrec_b200.distributed.planner.partitioners import GreedyPerfPartitioner
    from torchrec_b200.inference.modules import quantize_inference_model, shard_quant_model
    from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection, EmbeddingCollection
    from torchrec_b200.optim.keyed import CombinedOptimizer, KeyedOptimizer, KeyedOptimizerWrapper
    from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor, KeyedTensor

    R = "required"
    return {
        "DMP.__init__": (DistributedModelParallel.__init__, [("module", R), ("env", None), ("device", None), ("plan", None), ("sharders", None),
                                                             ("init_data_parallel", True), ("init_parameters", True), ("data_parallel_wrapper", None)]),
        "EBC.__init__": (EmbeddingBagCollection.__init__, [("tables", R), ("is_weighted", False), ("device", None)]),
        "EBC.forward": (EmbeddingBagCollection.forward, [("features", R)]),
        "EC.__init__": (EmbeddingCollection.__init__, [("tables", R), ("device", None), ("need_indices", False)]),
        "EC.forward": (EmbeddingCollection.forward, [("features", R)]),
        "Planner.__init__": (EmbeddingShardingPlanner.__init__, [("topology", None), ("batch_size", None), ("enumerator", None), ("storage_reservation", None),
                                                                 ("proposer", None), ("partitioner", None), ("performance_model", None), ("stats", None),
                                                                 ("constraints", None), ("debug", True)]),
        "Planner.collective_plan": (EmbeddingShardingPlanner.collective_plan, [("module", R), ("sharders", None), ("pg", None)]),
        "Planner.plan": (EmbeddingShardingPlanner.plan, [("module", R), ("sharders", R)]),
        "Enumerator.__init__": (EmbeddingEnumerator.__init__, [("topology", R), ("batch_size", R), ("constraints", None), ("estimator", None),
                                                               ("use_exact_enumerate_order", False)]),
        "Enumerator.enumerate": (EmbeddingEnumerator.enumerate, [("module", R), ("sharders", R)]),
        "Partitioner.__init__": (GreedyPerfPartitioner.__init__, [("sort_by", "any"), ("balance_modules", False)]),
        "JT.__init__": (JaggedTensor.__init__, [("values", R), ("weights", None), ("lengths", None), ("offsets", None)]),
        "KJT.__init__": (KeyedJaggedTensor.__init__, [("keys", R), ("values", R), ("weights", None), ("lengths", None), ("offsets", None), ("stride", None),
                                                      ("stride_per_key_per_rank", None)]),
        "KJT.from_lengths_sync": (KeyedJaggedTensor.from_lengths_sync, [("keys", R), ("values", R), ("lengths", R), ("weights", None)]),
        "KJT.from_offsets_sync": (KeyedJaggedTensor.from_offsets_sync, [("keys", R), ("values", R), ("offsets", R), ("weights", None)]),
        "KT.__init__": (KeyedTensor.__init__, [("keys", R), ("length_per_key", R), ("values", R), ("key_dim", 1)]),
        "KeyedOptimizer.__init__": (KeyedOptimizer.__init__, [("params", R), ("state", R), ("param_groups", R)]),
        "CombinedOptimizer.__init__": (CombinedOptimizer.__init__, [("optims", R)]),
        "KeyedOptimizerWrapper.__init__": (KeyedOptimizerWrapper.__init__, [("params", R), ("optim_factory", R)]),
        "quantize_inference_model": (quantize_inference_model, [("model", R), ("quantization_mapping", None)]),
        "shard_quant_model": (shard_quant_model, [("model", R), ("world_size", 1), ("compute_device", "cuda"), ("sharding_device", "meta"), ("sharders", None)]),
    }


@pytest.mark.parametrize("name", sorted(_cases()))
def test_signature_is_call_compatible(name):
    fn, expected = _cases()[name]
    params = [p for p in inspect.signature(fn).parameters.values() if p.name not in ("self", "cls")]
    names = [p.name for p in params]
    pos = -1
    for pname, default in expected:
        assert pname in names, f"{name}: parameter {pname} missing (has {names})"
        idx = names.index(pname)
        assert idx > pos, f"{name}: parameter {pname} out of order"
        pos = idx
        has_default = params[idx].default is not inspect.Parameter.empty
        if default != "required":
            assert has_default, f"{name}: {pname} must stay optional"
            if default != "any":
                assert params[idx].default == default, f"{name}: default of {pname} is {params[idx].default!r}, expected {default!r}"
    # parameters added here beyond the reference's must not be required
    for p in params:
        if p.name not in [e[0] for e in expected] and p.kind in (p.POSITIONAL_OR_KEYWORD, p.KEYWORD_ONLY):
            assert p.default is not inspect.Parameter.empty, f"{name}: extra parameter {p.name} has no default"


def test_package_level_exports():
    import torchrec_b200 as t
    import torchrec_b200.distributed as d

    for name in ("DataType", "EmbeddingBagConfig", "EmbeddingConfig", "PoolingType", "EmbeddingBagCollection", "EmbeddingBagCollectionInterface", "EmbeddingCollection",
                 "JaggedTensor", "KeyedJaggedTensor", "KeyedTensor", "Multistreamable", "Pipelineable", "__version__", "distributed", "quant", "tracer"):
        assert getattr(t, name) is not None, name
    for name in ("get_local_rank", "get_local_size", "DistributedModelParallel", "DataLoadingThread", "EvalPipelineSparseDist", "PrefetchTrainPipelineSparseDist",
                 "TrainPipeline", "TrainPipelineBase", "TrainPipelineSparseDist", "Awaitable", "ModuleSharder", "NoWait", "ParameterSharding", "ShardedModule",
                 "ShardedTensor", "ShardingEnv", "ShardingPlanner", "get_unsharded_module_names", "sharded_model_copy"):
        assert getattr(d, name) is not None, name
