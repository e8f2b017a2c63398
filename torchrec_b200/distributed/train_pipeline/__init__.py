"""Training pipelines that overlap host-to-device copies, sparse input distribution and compute
(cf. ``torchrec/distributed/train_pipeline/__init__.py``)."""
from torchrec_b200.distributed.train_pipeline.pipeline_context import (  # noqa: F401
    EmbeddingTrainPipelineContext,
    PrefetchTrainPipelineContext,
    TrainPipelineContext,
)
from torchrec_b200.distributed.train_pipeline.train_pipelines import (  # noqa: F401
    EvalPipelineSparseDist,
    PrefetchTrainPipelineSparseDist,
    StagedTrainPipeline,
    TrainPipeline,
    TrainPipelineBase,
    TrainPipelineFusedSparseDist,
    TrainPipelinePT2,
    TrainPipelineSemiSync,
    TrainPipelineSparseDist,
    TrainPipelineSparseDistCompAutograd,
)
from torchrec_b200.distributed.train_pipeline.types import ArgInfo, CallArgs, PipelineState  # noqa: F401
from torchrec_b200.distributed.train_pipeline.utils import DataLoadingThread, In, Out, _to_device, _wait_for_batch  # noqa: F401
from torchrec_b200.distributed.train_pipeline.postproc import PipelinedPostproc  # noqa: F401
from torchrec_b200.distributed.train_pipeline.graphed import TrainPipelineGraphed  # noqa: F401
