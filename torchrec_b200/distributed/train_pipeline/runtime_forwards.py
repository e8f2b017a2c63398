"""Replacement ``forward`` callables installed on sharded modules by the pipelines: the input dist was
started ahead of time, so ``forward`` only waits for it and runs ``compute_and_output_dist``.
Counterpart of ``torchrec/distributed/train_pipeline/runtime_forwards.py``.
"""
from __future__ import annotations

import logging
from typing import Any, Callable, Dict, Generic, List, Optional, Tuple, TypeVar

import torch
from torch.autograd.profiler import record_function

from torchrec_b200.distributed.train_pipeline.pipeline_context import (
    EmbeddingTrainPipelineContext,
    PrefetchTrainPipelineContext,
    TrainPipelineContext,
)
from torchrec_b200.distributed.train_pipeline.types import CallArgs
from torchrec_b200.distributed.types import Awaitable, LazyNoWait, ShardedModule
from torchrec_b200.streamable import Multistreamable

logger: logging.Logger = logging.getLogger(__name__)
TForwardContext = TypeVar("TForwardContext", bound=TrainPipelineContext)


class BaseForward(Generic[TForwardContext]):
    def __init__(self, name: str, args: CallArgs, module: ShardedModule, context: TForwardContext, stream: Optional[torch.Stream] = None) -> None:
        self._name = name
        self._args = args
        self._module = module
        self._context = context
        self._stream = stream
        self._device: torch.device = stream.device if stream else torch.device("cpu")
        self._original_forward = module.forward

    @property
    def name(self) -> str:
        return self._name

    @property
    def args(self) -> CallArgs:
        return self._args

    def set_context(self, context: TForwardContext) -> None:
        self._context = context

    def get_context(self) -> TForwardContext:
        return self._context


class PipelinedForward(BaseForward[TrainPipelineContext]):
    """Waits for the pre-started input dist of this batch, then computes and starts the output dist."""

    def __call__(self, *input, **kwargs) -> Awaitable:
        if self._name not in self._context.input_dist_tensors_requests:
            # nothing was started for this batch (first batch, or called outside the pipeline)
            return self._original_forward(*input, **kwargs)
        request = self._context.input_dist_tensors_requests.pop(self._name)
        assert isinstance(request, Awaitable)
        with record_function("## wait_sparse_data_dist ##"):
            if self._stream is not None:
                with torch.get_device_module(self._device).stream(self._stream):
                    data = request.wait()
            else:
                data = request.wait()
        ctx = self._context.module_contexts.pop(self._name)
        if self._stream is not None:
            cur_stream = torch.get_device_module(self._device).current_stream()
            cur_stream.wait_stream(self._stream)
            assert isinstance(data, (torch.Tensor, Multistreamable)), f"{type(data)} must implement Multistreamable interface"
            data.record_stream(cur_stream)
            ctx.record_stream(cur_stream)
        return self._module.compute_and_output_dist(ctx, data)


class EmbeddingPipelinedForward(BaseForward[EmbeddingTrainPipelineContext]):
    """For pipelines that also run the lookup ahead of time: returns the pre-started output awaitable."""

    def __call__(self, *input, **kwargs) -> Awaitable:
        if self._name not in self._context.embedding_a2a_requests:
            return self._original_forward(*input, **kwargs)
        ctx = self._context.module_contexts.pop(self._name) if self._name in self._context.module_contexts else None
        cur_stream = torch.get_device_module(self._device).current_stream() if self._stream is not None else None
        if self._stream is not None and cur_stream is not None:
            cur_stream.wait_stream(self._stream)
            if ctx is not None:
                ctx.record_stream(cur_stream)
        return self._context.embedding_a2a_requests.pop(self._name)


class InSyncEmbeddingPipelinedForward(EmbeddingPipelinedForward):
    """Same as ``EmbeddingPipelinedForward``; the lookup it returns was computed with current weights."""


class PrefetchPipelinedForward(BaseForward[PrefetchTrainPipelineContext]):
    """Uses inputs that already went through the prefetch stage."""

    def __init__(self, name: str, args: CallArgs, module: ShardedModule, context: PrefetchTrainPipelineContext, prefetch_stream: Optional[torch.Stream] = None) -> None:
        super().__init__(name, args, module, context, prefetch_stream)

    def __call__(self, *input, **kwargs) -> Awaitable:
        if self._name not in self._context.module_input_post_prefetch:
            return self._original_forward(*input, **kwargs)
        data = self._context.module_input_post_prefetch.pop(self._name)
        ctx = self._context.module_contexts_post_prefetch.pop(self._name)
        if self._stream is not None:
            cur_stream = torch.get_device_module(self._device).current_stream()
            cur_stream.wait_stream(self._stream)
            data.record_stream(cur_stream)
            ctx.record_stream(cur_stream)
        return self._module.compute_and_output_dist(ctx, data)


class PrefetchEmbeddingPipelinedForward(PrefetchPipelinedForward):
    """For a pipeline that prefetches AND runs the lookup of batch N at the end of step N - 1: the pipeline calls
    ``compute_and_output_dist()`` ahead of time (on the inputs that went through the prefetch stage) and the model's forward then only
    picks up the awaitable.  Calling the forward first is a usage error
    (``torchrec/distributed/train_pipeline/runtime_forwards.py:271-328``)."""

    def __init__(self, name: str, args: CallArgs, module: ShardedModule, context: PrefetchTrainPipelineContext, prefetch_stream: Optional[torch.Stream] = None) -> None:
        super().__init__(name, args, module, context, prefetch_stream)
        self._compute_and_output_dist_awaitable: Optional[Awaitable] = None

    def compute_and_output_dist(self) -> None:
        assert self._name in self._context.module_input_post_prefetch, (
            "PrefetchEmbeddingPipelinedForward has no prefetched input for this module: do not call model.forward() directly")
        data = self._context.module_input_post_prefetch.pop(self._name)
        ctx = self._context.module_contexts_post_prefetch.pop(self._name)
        if self._stream is not None:
            cur_stream = torch.get_device_module(self._device).current_stream()
            cur_stream.wait_stream(self._stream)
            data.record_stream(cur_stream)
            ctx.record_stream(cur_stream)
        self._compute_and_output_dist_awaitable = self._module.compute_and_output_dist(ctx, data)

    def __call__(self, *input, **kwargs) -> Awaitable:
        if self._compute_and_output_dist_awaitable is None:
            raise Exception("compute_and_output_dist must be called before __call__")
        out, self._compute_and_output_dist_awaitable = self._compute_and_output_dist_awaitable, None
        return out


class KJTAllToAllForward:
    """Stage 1 of ``KJTAllToAll`` without the collective: the pipelines batch the split exchange of all
    modules into one collective (``FusedKJTListSplitsAwaitable``)."""

    def __init__(self, pg, splits: List[int], stagger: int = 1) -> None:
        self._pg = pg
        self._splits = splits
        self._stagger = stagger
        self._splits_cumsum = [0]
        for s in splits:
            self._splits_cumsum.append(self._splits_cumsum[-1] + s)

    def __call__(self, input):
        from torchrec_b200.distributed.dist_data import KJTAllToAllSplitsAwaitable

        with torch.no_grad():
            assert len(input.keys()) == sum(self._splits)
            rank = self._pg.rank()
            local_keys = input.keys()[self._splits_cumsum[rank]: self._splits_cumsum[rank + 1]]
            return KJTAllToAllSplitsAwaitable(
                pg=self._pg, input=input, splits=self._splits, labels=input.dist_labels(), tensor_splits=input.dist_splits(self._splits),
                input_tensors=input.dist_tensors(), keys=local_keys, device=input.device(), stagger=self._stagger,
            )
