"""Argument discovery for the sparse-dist pipelines: which attribute path of the batch (or of a post-processing module's output) each
sharded module's inputs come from.

The counterpart (``torchrec/distributed/train_pipeline/tracing.py:40-588``) symbolically traces the model with fx and walks the graph
backwards from every sharded module call.  Here the first batch runs unpipelined with hooks that record the actual arguments, and
``ArgRecorder.resolve`` locates those objects inside the batch by identity -- no tracer, so models with data-dependent control flow
pipeline as well.  The pieces live in ``utils.py``; this module is their import path under the counterpart's name."""
from torchrec_b200.distributed.train_pipeline.postproc import PipelinedPostproc  # noqa: F401
from torchrec_b200.distributed.train_pipeline.types import (  # noqa: F401
    ArgInfo,
    ArgInfoStepFactory,
    BaseArgInfoStep,
    CallArgs,
    DictArgInfoStep,
    GetAttrArgInfoStep,
    GetItemArgInfoStep,
    ListArgInfoStep,
    NoopArgInfoStep,
    PostprocArgInfoStep,
    ScalarArgInfoStep,
)
from torchrec_b200.distributed.train_pipeline.utils import (  # noqa: F401
    ArgRecorder,
    _find_path,
    find_postproc_candidates,
    find_sharded_modules,
)
