"""Benchmark builders end to end on two gloo ranks: config -> model -> planner -> sharded model + optimizer -> pipeline -> steps."""
import pytest
import torch

from torchrec_b200.test_utils.multi_process import MultiProcessContext, run_multi_process


def _run(rank, world_size, model_name, pipeline):
    from torchrec_b200.distributed.benchmark.benchmark_utils import (
        create_model_config, generate_data, generate_pipeline, generate_planner, generate_sharded_model_and_optimizer,
    )
    from torchrec_b200.distributed.embedding_types import EmbeddingComputeKernel
    from torchrec_b200.distributed.planner import Topology
    from torchrec_b200.distributed.types import ShardingType
    from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig

    with MultiProcessContext(rank, world_size, "gloo") as ctx:
        torch.manual_seed(0)
        tables = [EmbeddingBagConfig(name=f"t{i}", embedding_dim=16, num_embeddings=100, feature_names=[f"f{i}"]) for i in range(4)]
        cfg = create_model_config(model_name, batch_size=8, num_float_features=6, feature_pooling_avg=3, pin_memory=False,
                                  dense_arch_layer_sizes=[8, 16], over_arch_layer_sizes=[8, 1])
        model = cfg.generate_model(tables, [], torch.device("cpu"))
        planner = generate_planner("embedding", Topology(world_size=world_size, compute_device="cpu"), tables, None, ShardingType.TABLE_WISE,
                                   EmbeddingComputeKernel.FUSED, batch_sizes=[8])
        dmp, opt = generate_sharded_model_and_optimizer(model, ShardingType.TABLE_WISE.value, EmbeddingComputeKernel.FUSED.value, ctx.pg, torch.device("cpu"),
                                                        fused_params={"learning_rate": 0.05}, planner=planner)
        data = generate_data(tables, [], cfg, [8] * 5)
        pipe = generate_pipeline(pipeline, "data_dist", dmp, opt, torch.device("cpu"))
        it = iter(data)
        outs = [pipe.progress(it) for _ in range(5)]
        assert all(torch.isfinite(o[0] if isinstance(o, tuple) else o).all() for o in outs)
        with pytest.raises(RuntimeError):
            generate_pipeline("nope", "data_dist", dmp, opt, torch.device("cpu"))


@pytest.mark.parametrize("model_name,pipeline", [("dlrm", "sparse"), ("deepfm", "base"), ("test_sparse_nn", "sparse")])
def test_benchmark_builders(model_name, pipeline):
    run_multi_process(_run, world_size=2, model_name=model_name, pipeline=pipeline)
