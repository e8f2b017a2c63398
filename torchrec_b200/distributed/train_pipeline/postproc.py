"""Pipelined input post-processing.

A module that sits between the batch and a sharded embedding module (id remapping, feature slicing, ...) would force the input
dist of that embedding module to wait for the model forward.  ``PipelinedPostproc`` takes the module's place in the model: the
pipeline runs it for batch ``i + 1`` on the data-dist stream while batch ``i`` trains, caches the result in that batch's context,
and the model forward of batch ``i + 1`` gets the cached result instead of running the module again.
Counterpart of ``torchrec/distributed/train_pipeline/postproc.py:40-250``."""
from __future__ import annotations

from typing import Any, Optional

import torch
from torch.profiler import record_function

from torchrec_b200.distributed.train_pipeline.pipeline_context import TrainPipelineContext
from torchrec_b200.distributed.train_pipeline.types import CallArgs


def _record_stream(obj: Any, stream: torch.Stream, depth: int = 0) -> None:
    if depth > 4:
        return
    if isinstance(obj, torch.Tensor):
        if obj.is_cuda:
            obj.record_stream(stream)
    elif hasattr(obj, "record_stream"):
        obj.record_stream(stream)
    elif isinstance(obj, (list, tuple)):
        for v in obj:
            _record_stream(v, stream, depth + 1)
    elif isinstance(obj, dict):
        for v in obj.values():
            _record_stream(v, stream, depth + 1)


class NoOpStream:
    """Context manager that accepts a stream and does nothing: stands in for ``torch.cuda.stream(...)`` where there is no stream to
    switch to (CPU runs, or a post-processing module that stays on the caller's stream)."""

    def __init__(self, stream: Optional[torch.Stream]) -> None:
        self._stream = stream

    def __enter__(self) -> "NoOpStream":
        return self

    def __exit__(self, exc_type, exc_value, traceback) -> None:
        return None


class PipelinedPostproc(torch.nn.Module):
    """Stands in for ``postproc_module`` (found at ``fqn`` in the model).  ``run(batch, context)`` computes the module's output
    from the batch through ``call_args`` once per context; ``forward`` returns the output cached in the current context, or falls
    back to calling the module on the arguments it was given when nothing is cached (first batches, evaluation outside the
    pipeline)."""

    def __init__(self, postproc_module: torch.nn.Module, fqn: str, call_args: CallArgs, context: Optional[TrainPipelineContext] = None) -> None:
        super().__init__()
        self._postproc_module = postproc_module
        self._fqn = fqn
        self._call_args = call_args
        self._context = context
        if any(p.requires_grad for p in postproc_module.parameters()):
            raise ValueError(f"post-processing module {fqn} has trainable parameters and cannot run ahead of the step")

    @property
    def postproc_module(self) -> torch.nn.Module:
        return self._postproc_module

    @property
    def fqn(self) -> str:
        return self._fqn

    def set_context(self, context: TrainPipelineContext) -> None:
        self._context = context

    def get_context(self) -> Optional[TrainPipelineContext]:
        return self._context

    def run(self, batch: Any, context: Optional[TrainPipelineContext]) -> Any:
        """Output for ``batch``, computed at most once per ``context`` (call on the stream the consumers run on)."""
        ctx = context if context is not None else self._context
        if ctx is not None and self._fqn in ctx.postproc_fwd_results:
            return ctx.postproc_fwd_results[self._fqn]
        with record_function(f"## pipelined postproc {self._fqn} ##"):
            args, kwargs = self._call_args.build_args_kwargs(batch, ctx)
            out = self._postproc_module(*args, **kwargs)
        if ctx is not None:
            ctx.postproc_fwd_results[self._fqn] = out
        return out

    def forward(self, *args: Any, **kwargs: Any) -> Any:
        ctx = self._context
        if ctx is not None and self._fqn in ctx.postproc_fwd_results:
            out = ctx.postproc_fwd_results[self._fqn]
            if torch.cuda.is_available() and torch.cuda.is_initialized():
                # produced on the data-dist stream, consumed on the stream of the model forward
                _record_stream(out, torch.cuda.current_stream())
            return out
        return self._postproc_module(*args, **kwargs)
