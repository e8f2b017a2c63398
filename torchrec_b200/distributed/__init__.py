"""Sharding runtime: ``DistributedModelParallel``, sharded modules, planner, train pipelines.

Mirrors the export surface of ``torchrec/distributed/__init__.py:33-60``.
"""
from torchrec_b200.distributed.comm import get_local_rank, get_local_size  # noqa: F401
from torchrec_b200.distributed.types import (  # noqa: F401
    Awaitable,
    LazyAwaitable,
    ModuleSharder,
    NoWait,
    ParameterSharding,
    ShardedModule,
    ShardedTensor,
    ShardingEnv,
    ShardingPlan,
    ShardingPlanner,
    ShardingType,
)
from torchrec_b200.distributed.utils import get_unsharded_module_names, sharded_model_copy  # noqa: F401


def __getattr__(name):
    # heavier modules are imported on first use to keep `import torchrec_b200.distributed` cheap and acyclic
    if name in ("DistributedModelParallel", "DMPCollection"):
        from torchrec_b200.distributed import model_parallel

        return getattr(model_parallel, name)
    if name in ("TrainPipeline", "TrainPipelineBase", "TrainPipelineSparseDist", "TrainPipelineFusedSparseDist", "TrainPipelineSemiSync",
                "PrefetchTrainPipelineSparseDist", "EvalPipelineSparseDist", "StagedTrainPipeline", "DataLoadingThread", "PipelinedPostproc"):
        from torchrec_b200.distributed import train_pipeline
        return getattr(train_pipeline, name)
    raise AttributeError(name)
