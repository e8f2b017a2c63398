"""Per-batch state carried through the pipeline stages
(cf. ``torchrec/distributed/train_pipeline/pipeline_context.py``)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch

from torchrec_b200.distributed.embedding_sharding import FusedKJTListSplitsAwaitable
from torchrec_b200.distributed.types import Awaitable, LazyAwaitable
from torchrec_b200.streamable import Multistreamable


@dataclass
class TrainPipelineContext:
    """State of one in-flight batch.

    ``input_dist_splits_requests``: stage-1 awaitables by module name (after ``start_sparse_data_dist``);
    ``input_dist_tensors_requests``: stage-2 awaitables (after ``wait_sparse_data_dist``);
    ``module_contexts``: the sharded modules' own contexts for this batch.
    """

    input_dist_splits_requests: Dict[str, Awaitable[Any]] = field(default_factory=dict)
    input_dist_tensors_requests: Dict[str, Awaitable[Any]] = field(default_factory=dict)
    module_contexts: Dict[str, Multistreamable] = field(default_factory=dict)
    module_contexts_next_batch: Dict[str, Multistreamable] = field(default_factory=dict)
    fused_splits_awaitables: List[Any] = field(default_factory=list)
    event: Optional[torch.Event] = None
    postproc_fwd_results: Dict[str, Any] = field(default_factory=dict)
    index: Optional[int] = None
    version: int = 1


@dataclass
class PrefetchTrainPipelineContext(TrainPipelineContext):
    module_input_post_prefetch: Dict[str, Multistreamable] = field(default_factory=dict)
    module_contexts_post_prefetch: Dict[str, Multistreamable] = field(default_factory=dict)
    module_input_post_prefetch_next_batch: Dict[str, Multistreamable] = field(default_factory=dict)
    module_contexts_post_prefetch_next_batch: Dict[str, Multistreamable] = field(default_factory=dict)


@dataclass
class EmbeddingTrainPipelineContext(TrainPipelineContext):
    embedding_a2a_requests: Dict[str, Any] = field(default_factory=dict)
    embedding_tensors: List[List[torch.Tensor]] = field(default_factory=list)
    embedding_features: List[List[Any]] = field(default_factory=list)
    detached_embedding_tensors: List[List[torch.Tensor]] = field(default_factory=list)
