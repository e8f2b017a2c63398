"""Stages for ``StagedTrainPipeline`` (cf. ``torchrec/distributed/train_pipeline/pipeline_stage.py``)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional

import torch

from torchrec_b200.distributed.train_pipeline.pipeline_context import TrainPipelineContext
from torchrec_b200.distributed.train_pipeline.types import CallArgs
from torchrec_b200.distributed.train_pipeline.utils import ArgRecorder, _start_data_dist, _wait_data_dist, find_sharded_modules
from torchrec_b200.distributed.types import ShardedModule


@dataclass
class PipelineStage:
    """One stage: ``runnable(batch) -> batch`` executed on ``stream``."""

    name: str
    runnable: Callable[[Any], Any]
    stream: Optional[torch.Stream] = None
    fill_callback: Optional[Callable[[], None]] = None


class SparseDataDistUtil:
    """Runs the sparse input dist of the sharded modules as two pipeline stages
    (``start_sparse_data_dist`` / ``wait_sparse_data_dist``) of a ``StagedTrainPipeline``.

    The batch fields that each sharded module consumes are discovered from the first model forward
    (call ``observe(batch)`` with the batch about to be run, then run the model once).
    """

    def __init__(self, model: torch.nn.Module, data_dist_stream: Optional[torch.Stream], apply_jit: bool = False, prefetch_stream: Optional[torch.Stream] = None) -> None:
        self.model = model
        self.data_dist_stream = data_dist_stream
        self.prefetch_stream = prefetch_stream
        self.context = TrainPipelineContext(version=1)
        self.initialized = False
        self._modules: Dict[str, ShardedModule] = find_sharded_modules(model)
        self._call_args: Dict[str, CallArgs] = {}
        self._recorder: Optional[ArgRecorder] = ArgRecorder(self._modules)
        self._first_batch: Any = None
        self._original_forwards: Dict[str, Any] = {}

    def observe(self, batch: Any) -> None:
        self._first_batch = batch

    def _maybe_init(self) -> bool:
        if self.initialized:
            return True
        if self._recorder is not None and self._recorder.calls and self._first_batch is not None:
            from torchrec_b200.distributed.train_pipeline.runtime_forwards import PipelinedForward

            self._call_args = self._recorder.resolve(self._first_batch)
            self._recorder.remove()
            self._recorder = None
            for name in self._call_args:
                m = self._modules[name]
                self._original_forwards[name] = m.forward
                m.forward = PipelinedForward(name, self._call_args[name], m, self.context, self.data_dist_stream)  # type: ignore[assignment]
            self.initialized = True
        return self.initialized

    def start_sparse_data_dist(self, batch: Any) -> Any:
        if not self._maybe_init():
            if self._first_batch is None:
                self._first_batch = batch
            return batch
        _start_data_dist({n: self._modules[n] for n in self._call_args}, self._call_args, batch, self.context)
        return batch

    def wait_sparse_data_dist(self, batch: Any) -> Any:
        if self.initialized:
            _wait_data_dist(self.context)
        return batch

    def detach(self) -> torch.nn.Module:
        for name, fwd in self._original_forwards.items():
            self._modules[name].forward = fwd  # type: ignore[assignment]
        self.initialized = False
        return self.model
