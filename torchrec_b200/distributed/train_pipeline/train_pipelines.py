"""Train pipelines: software pipelining of *batches* across CUDA streams.

* ``TrainPipelineBase``: copy batch i+1 to the device while batch i trains.
* ``TrainPipelineSparseDist``: additionally run the sparse input dist (KJT all-to-all) of batch i+1
  on a side stream during the forward/backward of batch i, and copy batch i+2.
* ``TrainPipelineFusedSparseDist``: also run the embedding lookup of batch i+1 ahead of time on its own
  stream (valid because the fused optimizer has already updated the tables when it is launched).
* ``TrainPipelineSemiSync``: start batch i+1's embedding lookup + output dist before batch i's
  backward (embeddings are one step stale), with a separate embedding backward.
* ``PrefetchTrainPipelineSparseDist``: adds a prefetch stage for cached tables.
* ``EvalPipelineSparseDist``: forward only.  ``StagedTrainPipeline``: user-defined stages.

Counterpart of ``torchrec/distributed/train_pipeline/train_pipelines.py:104-2106``.
"""
from __future__ import annotations

import abc
import contextlib
import logging
from collections import deque
from dataclasses import dataclass
from typing import Any, Callable, Deque, Dict, Generic, Iterator, List, Optional, Tuple, Type, Union, cast

import torch
from torch.autograd.profiler import record_function

from torchrec_b200.distributed.dist_data import KJTAllToAll
from torchrec_b200.distributed.model_parallel import DistributedModelParallel
from torchrec_b200.distributed.train_pipeline.pipeline_context import (
    EmbeddingTrainPipelineContext,
    PrefetchTrainPipelineContext,
    TrainPipelineContext,
)
from torchrec_b200.distributed.train_pipeline.runtime_forwards import (
    EmbeddingPipelinedForward,
    InSyncEmbeddingPipelinedForward,
    PipelinedForward,
    PrefetchPipelinedForward,
)
from torchrec_b200.distributed.train_pipeline.types import CallArgs, PipelineState
from torchrec_b200.distributed.train_pipeline.utils import (
    ArgRecorder,
    find_postproc_candidates,
    DataLoadingThread,
    In,
    Out,
    _start_data_dist,
    _to_device,
    _wait_data_dist,
    _wait_for_batch,
    find_sharded_modules,
)
from torchrec_b200.distributed.types import Awaitable, ShardedModule
from torchrec_b200.streamable import Multistreamable, Pipelineable

logger: logging.Logger = logging.getLogger(__name__)


class ModelDetachedException(Exception):
    pass


@dataclass
class TorchCompileConfig:
    """Compile settings in the shape ``TrainPipelinePT2`` accepts: whole-graph capture, dynamic shapes (None: automatic), backend,
    and the iteration at which compilation would happen.  No pipeline of this package compiles the model (the hot path is the
    hand-written kernels); only ``compile_on_iter`` has an effect: it is the iteration at which the pre / post compile hooks run."""

    fullgraph: bool = False
    dynamic: Optional[bool] = None
    backend: str = "inductor"
    compile_on_iter: int = 3


class TrainPipeline(abc.ABC, Generic[In, Out]):
    @abc.abstractmethod
    def progress(self, dataloader_iter: Iterator[In]) -> Out:
        ...

    def sync_embeddings(self, model: torch.nn.Module, interval_batches: Optional[int], context: Optional[TrainPipelineContext] = None) -> None:
        """2D parallelism: average embedding replicas every ``interval_batches`` steps."""
        from torchrec_b200.distributed.model_parallel import DMPCollection

        if not isinstance(model, DMPCollection) or interval_batches is None:
            return
        index = context.index if context is not None and context.index is not None else 0
        if (index + 1) % interval_batches == 0:
            with record_function("## dmp_collection_sync ##"):
                model.sync()

    def reset(self) -> None:
        pass


def _device_streams(device: torch.device, n: int) -> List[Optional[torch.Stream]]:
    """``n`` high-priority side streams on an accelerator, ``None`` placeholders on the CPU."""
    if device.type in ("cuda", "mtia"):
        mod = torch.get_device_module(device)
        return [mod.Stream(priority=-1) if device.type == "cuda" else mod.Stream() for _ in range(n)]
    return [None] * n


def _stream_scope(device: torch.device):
    return torch.get_device_module(device).stream if device.type in ("cuda", "mtia") else contextlib.nullcontext


class TrainPipelineBase(TrainPipeline[In, Out]):
    """Two-deep pipeline: host-to-device copy of the next batch overlaps the current step."""

    def __init__(self, model: torch.nn.Module, optimizer: torch.optim.Optimizer, device: torch.device, custom_model_fwd: Optional[Callable[[In], Tuple[torch.Tensor, Out]]] = None) -> None:
        self._model, self._optimizer, self._device = model, optimizer, device
        (self._memcpy_stream,) = _device_streams(device, 1)
        self._stream_context = _stream_scope(device)
        self._model_fwd: Callable[[In], Tuple[torch.Tensor, Out]] = custom_model_fwd or model
        self._reset_data_iter()

    def _reset_data_iter(self) -> None:
        self._connected, self._data_iter_stopped, self._cur_batch = False, False, None

    def _next_batch(self, dataloader_iter: Iterator[In]) -> Optional[In]:
        with record_function("## next_batch ##"):
            batch = next(dataloader_iter, None)
        self._data_iter_stopped = batch is None
        return batch

    def _copy_batch_to_gpu(self, cur_batch: In) -> None:
        with record_function("## copy_batch_to_gpu ##"), self._stream_context(self._memcpy_stream):
            self._cur_batch = _to_device(cur_batch, self._device, non_blocking=True)

    def _connect(self, dataloader_iter: Iterator[In]) -> None:
        self._copy_batch_to_gpu(next(dataloader_iter))
        self._connected = True

    def _wait_for_batch(self, cur_batch: In) -> None:
        with record_function("## wait_for_batch ##"):
            _wait_for_batch(cur_batch, self._memcpy_stream)

    def _backward(self, losses: torch.Tensor) -> None:
        with record_function("## backward ##"):
            torch.sum(losses, dim=0).backward()

    def progress(self, dataloader_iter: Iterator[In]) -> Out:
        if not self._connected:
            self._connect(dataloader_iter)
        if self._data_iter_stopped:
            raise StopIteration()
        batch = cast(In, self._cur_batch)
        training = self._model.training
        if training:
            with record_function("## zero_grad ##"):
                self._optimizer.zero_grad()
        self._wait_for_batch(batch)
        upcoming = self._next_batch(dataloader_iter)  # fetched now so that the loader works while the device computes
        with record_function("## forward ##"):
            losses, output = self._model_fwd(batch)
        if training:
            self._backward(losses)
        if upcoming is None:
            self._cur_batch = None
        else:
            self._copy_batch_to_gpu(upcoming)
        if training:
            with record_function("## optimizer ##"):
                self._optimizer.step()
        return output


class TrainPipelinePT2(TrainPipelineBase[In, Out]):
    """Kept for API parity: this framework does not use a tracing compiler, so the model runs eagerly
    (CUDA kernels + streams); the class behaves like ``TrainPipelineBase``.  The captured-step counterpart is
    ``TrainPipelineGraphed``.  ``pre_compile_fn`` / ``post_compile_fn`` run once, at iteration ``compile_configs.compile_on_iter``
    (where the counterpart compiles, ``torchrec/distributed/train_pipeline/train_pipelines.py:329-372``)."""

    def __init__(self, model: torch.nn.Module, optimizer: torch.optim.Optimizer, device: torch.device,
                 compile_configs: Optional[TorchCompileConfig] = None,
                 pre_compile_fn: Optional[Callable[[torch.nn.Module], None]] = None, post_compile_fn: Optional[Callable[[torch.nn.Module], None]] = None,
                 input_transformer: Optional[Callable[[In], In]] = None) -> None:
        super().__init__(model, optimizer, device)
        self._compile_configs: TorchCompileConfig = compile_configs or TorchCompileConfig()
        self._pre_compile_fn = pre_compile_fn
        self._post_compile_fn = post_compile_fn
        self._input_transformer = input_transformer
        self._iter = 0

    def progress(self, dataloader_iter: Iterator[In]) -> Out:
        if self._iter == self._compile_configs.compile_on_iter:
            for hook in (self._pre_compile_fn, self._post_compile_fn):
                if hook is not None:
                    hook(self._model)
        self._iter += 1
        transform = self._input_transformer
        return super().progress(dataloader_iter if transform is None else map(transform, dataloader_iter))


class TrainPipelineSparseDist(TrainPipeline[In, Out]):
    """Three batches in flight: batch i trains, batch i+1's sparse input dist runs on ``data_dist_stream``,
    batch i+2 is copied on ``memcpy_stream``.

    Args:
        model: model containing sharded modules (usually a ``DistributedModelParallel``).
        optimizer: optimizer stepped after backward (fused embedding optimizers only sync their LR).
        device: device of this rank.
        execute_all_batches: keep stepping until the in-flight batches are drained when the data ends.
        apply_jit / enqueue_batch_after_forward / context_type / custom_model_fwd / dmp_collection_sync_interval_batches: as named.

    A step is a fixed sequence of small phases (``_step_*`` methods); the derived pipelines change single phases instead of
    re-stating the loop.
    """

    _model_attached: bool = True

    def __init__(self, model: torch.nn.Module, optimizer: torch.optim.Optimizer, device: torch.device, execute_all_batches: bool = True,
                 apply_jit: bool = False, context_type: Type[TrainPipelineContext] = TrainPipelineContext,
                 pipeline_postproc: bool = False, custom_model_fwd: Optional[Callable[[Optional[In]], Tuple[torch.Tensor, Out]]] = None,
                 dmp_collection_sync_interval_batches: Optional[int] = 1, enqueue_batch_after_forward: bool = False) -> None:
        self._model, self._optimizer, self._device = model, optimizer, device
        self._execute_all_batches = execute_all_batches
        self._apply_jit = apply_jit
        self._enqueue_batch_after_forward = enqueue_batch_after_forward
        self._pipeline_postproc = pipeline_postproc
        self._dmp_collection_sync_interval_batches = dmp_collection_sync_interval_batches
        self._memcpy_stream, self._data_dist_stream = _device_streams(device, 2) if device.type == "cuda" else (None, None)
        self._stream_context = _stream_scope(device)
        self._model_fwd: Callable[[Optional[In]], Tuple[torch.Tensor, Out]] = custom_model_fwd or model
        self._context_type = context_type
        self._context = context_type(version=0)
        # what pipelining changed in the model, so that detach() can undo it
        self._original_forwards: Dict[str, Callable[..., Any]] = {}
        self._pipelined_modules: Dict[str, ShardedModule] = {}
        self._pipelined_forwards: Dict[str, Any] = {}
        self._pipelined_postprocs: Dict[str, Any] = {}
        self._call_args: Dict[str, CallArgs] = {}
        self._recorder: Optional[ArgRecorder] = None
        self._pipelined: bool = False
        # batches in flight, oldest first, with their contexts
        self.batches: Deque[Optional[In]] = deque()
        self.contexts: Deque[TrainPipelineContext] = deque()
        self._batch_i = self._batch_ip1 = self._batch_ip2 = None
        self._dataloader_iter: Optional[Iterator[In]] = None
        self._dataloader_exhausted: bool = False
        self._next_index: int = 0
        self._state: PipelineState = PipelineState.IDLE

    # ---- batch queue -----------------------------------------------------------------------------------
    def _create_context(self) -> TrainPipelineContext:
        index, self._next_index = self._next_index, self._next_index + 1
        return self._context_type(index=index, version=1)

    def _next_batch(self, dataloader_iter: Iterator[In]) -> Optional[In]:
        """Next batch or None; a loader that ended once is not asked again (some loaders block on that)."""
        if self._dataloader_iter is not dataloader_iter:
            self._dataloader_iter, self._dataloader_exhausted = dataloader_iter, False
        if self._dataloader_exhausted:
            return None
        with record_function("## next_batch ##"):
            batch = next(dataloader_iter, None)
        self._dataloader_exhausted = batch is None
        return batch

    def copy_batch_to_gpu(self, dataloader_iter: Iterator[In]) -> Tuple[Optional[In], Optional[TrainPipelineContext]]:
        context = self._create_context()
        with record_function(f"## copy_batch_to_gpu {context.index} ##"), self._stream_context(self._memcpy_stream):
            batch = self._next_batch(dataloader_iter)
            if batch is None:
                if not self._execute_all_batches:
                    raise StopIteration
                return None, context
            return _to_device(batch, self._device, non_blocking=True), context

    def enqueue_batch(self, dataloader_iter: Iterator[In]) -> bool:
        batch, context = self.copy_batch_to_gpu(dataloader_iter)
        if batch is not None:
            self.batches.append(batch)
            self.contexts.append(cast(TrainPipelineContext, context))
        return batch is not None

    def dequeue_batch(self) -> None:
        self.batches.popleft()
        self.contexts.popleft()
        if self.contexts:
            self._set_module_context(self.contexts[0])

    def _set_module_context(self, context: TrainPipelineContext) -> None:
        for holder in (self._pipelined_forwards, self._pipelined_postprocs):
            for item in holder.values():
                item.set_context(context)

    # ---- pipelining the model --------------------------------------------------------------------------
    def _make_forward(self, name: str, module: ShardedModule, call_args: CallArgs, context: TrainPipelineContext):
        return PipelinedForward(name, call_args, module, context, self._data_dist_stream)

    def _install_recorder(self) -> None:
        self._all_sharded = find_sharded_modules(self._model)
        candidates = find_postproc_candidates(self._model, self._all_sharded) if self._pipeline_postproc else None
        self._recorder = ArgRecorder(self._all_sharded, candidates)

    @staticmethod
    def _defer_split_exchange(module: ShardedModule, defer: bool) -> None:
        for m in module.modules():
            if isinstance(m, KJTAllToAll):
                m.defer_splits_exchange = defer

    def _install_forwards(self, install: bool) -> None:
        """Put the pipelined forwards (and post-processing wrappers) into the model, or take them out again."""
        self._swap_postprocs(install)
        table = self._pipelined_forwards if install else self._original_forwards
        for name, module in self._pipelined_modules.items():
            module.forward = table[name]  # type: ignore[assignment]
            self._defer_split_exchange(module, install)
        self._pipelined = install

    def _pipeline_model(self, batch: In, context: TrainPipelineContext) -> None:
        """After the first (unpipelined) forward: resolve where every sharded module's inputs live in the
        batch and swap the modules' ``forward`` for pipelined ones."""
        recorder = self._recorder
        assert recorder is not None
        self._call_args = recorder.resolve(batch)
        recorder.remove()
        self._pipelined_postprocs = dict(recorder.postprocs)
        self._recorder = None
        for name, ca in self._call_args.items():
            module = self._all_sharded[name]
            self._pipelined_modules[name] = module
            self._original_forwards[name] = module.forward
            self._pipelined_forwards[name] = self._make_forward(name, module, ca, context)
        self._install_forwards(True)
        for pp in self._pipelined_postprocs.values():
            pp.set_context(context)

    def _swap_postprocs(self, install: bool) -> None:
        """Put the pipelined post-processing wrappers into the model in place of the modules they wrap, or take them out."""
        for fqn, pp in self._pipelined_postprocs.items():
            parent_name, _, child = fqn.rpartition(".")
            parent = self._model.get_submodule(parent_name) if parent_name else self._model
            setattr(parent, child, pp if install else pp.postproc_module)

    def detach(self) -> torch.nn.Module:
        """Restore the original forwards so the model can be used outside the pipeline."""
        if self._pipelined:
            self._install_forwards(False)
        self._model_attached = False
        return self._model

    def attach(self, model: Optional[torch.nn.Module] = None, sparse_dist: bool = True) -> None:
        if model is not None:
            self._model = model
        self._model_attached = True
        if not self._pipelined_forwards or self._pipelined:
            return
        self._install_forwards(True)
        if sparse_dist:
            # batches that were in flight lost their input dists on detach: run them again
            for batch, ctx in zip(self.batches, self.contexts):
                if not (ctx.input_dist_tensors_requests or ctx.input_dist_splits_requests):
                    self.start_sparse_data_dist(batch, ctx)
                    self.wait_sparse_data_dist(ctx)

    def start_sparse_data_dist(self, batch: Optional[In], context: TrainPipelineContext) -> None:
        """Stage 1 of the input dist of ``batch`` on the data-dist stream."""
        if batch is None or not self._pipelined:
            return
        with record_function(f"## start_sparse_data_dist {context.index} ##"), self._stream_context(self._data_dist_stream):
            _wait_for_batch(batch, self._memcpy_stream)
            _start_data_dist(self._pipelined_modules, self._call_args, batch, context)

    def wait_sparse_data_dist(self, context: TrainPipelineContext) -> None:
        """Finish stage 1 (host learns the split sizes) and launch stage 2."""
        if not self._pipelined:
            return
        with record_function(f"## wait_sparse_data_dist {context.index} ##"), self._stream_context(self._data_dist_stream):
            _wait_data_dist(context)

    def _wait_for_batch(self) -> None:
        producer = self._data_dist_stream if self._pipelined else self._memcpy_stream
        with record_function(f"## wait_for_batch {self.contexts[0].index} ##"):
            _wait_for_batch(cast(In, self.batches[0]), producer)

    def _backward(self, losses: torch.Tensor) -> None:
        with record_function(f"## backward {self.contexts[0].index} ##"):
            torch.sum(losses, dim=0).backward()

    def fill_pipeline(self, dataloader_iter: Iterator[In]) -> None:
        """Bring the queue to two batches (current + next), with the current one's input dist done."""
        have = len(self.batches)
        if have >= 2 or (have == 1 and self._execute_all_batches):
            return  # full, or draining the tail
        if not self.enqueue_batch(dataloader_iter):
            return
        if not (self._pipelined or self._recorder is not None or self._pipelined_forwards):
            self._install_recorder()
        if self._pipelined:
            head = self.contexts[0]
            self.start_sparse_data_dist(self.batches[0], head)
            self.wait_sparse_data_dist(head)
            self._set_module_context(head)
        self.enqueue_batch(dataloader_iter)

    # ---- one step, phase by phase -------------------------------------------------------------------------
    def _step_prepare(self, dataloader_iter: Iterator[In]) -> None:
        if not self._model_attached:
            self.attach(self._model)
        self.fill_pipeline(dataloader_iter)
        if not self.batches:
            raise StopIteration

    def _step_before_forward(self) -> None:
        """Hook between queue handling and the step proper (derived pipelines start look-ahead work here)."""

    def _step_open(self, dataloader_iter: Iterator[In]) -> None:
        self._state = PipelineState.IDLE
        if self._model.training:
            with record_function("## zero_grad ##"):
                self._optimizer.zero_grad()
        self._wait_for_batch()
        if self._pipelined and len(self.batches) >= 2:
            self.start_sparse_data_dist(self.batches[1], self.contexts[1])
        if not self._enqueue_batch_after_forward:
            self.enqueue_batch(dataloader_iter)

    def _step_forward(self, dataloader_iter: Iterator[In]) -> Tuple[torch.Tensor, Out]:
        self._state = PipelineState.CALL_FWD
        with record_function(f"## forward {self.contexts[0].index} ##"):
            losses, output = self._model_fwd(self.batches[0])
        if self._enqueue_batch_after_forward:
            self.enqueue_batch(dataloader_iter)
        if self._recorder is not None and not self._pipelined:
            # the first batch ran unpipelined; its recorded arguments tell where later batches' inputs come from
            self._pipeline_model(cast(In, self.batches[0]), self.contexts[min(1, len(self.contexts) - 1)])
            if len(self.batches) >= 2:
                self.start_sparse_data_dist(self.batches[1], self.contexts[1])
        return losses, output

    def _step_after_forward(self) -> None:
        if len(self.batches) >= 2:
            self.wait_sparse_data_dist(self.contexts[1])

    def _step_close(self, losses: torch.Tensor) -> None:
        if self._model.training:
            self._state = PipelineState.CALL_BWD
            self._backward(losses)
            self.sync_embeddings(self._model, self._dmp_collection_sync_interval_batches, self.contexts[0])
            with record_function(f"## optimizer {self.contexts[0].index} ##"):
                self._optimizer.step()
        self.dequeue_batch()

    def progress(self, dataloader_iter: Iterator[In]) -> Out:
        self._step_prepare(dataloader_iter)
        self._step_before_forward()
        self._step_open(dataloader_iter)
        losses, output = self._step_forward(dataloader_iter)
        self._step_after_forward()
        self._step_close(losses)
        return output

    def reset(self) -> None:
        self.batches.clear()
        self.contexts.clear()
        self._dataloader_iter, self._dataloader_exhausted = None, False


class TrainPipelineFusedSparseDist(TrainPipelineSparseDist[In, Out]):
    """Additionally starts the embedding lookup + output dist of the next batch on ``emb_lookup_stream``
    right after the previous optimizer step, so it overlaps the dense forward."""

    def __init__(self, model: torch.nn.Module, optimizer: torch.optim.Optimizer, device: torch.device, execute_all_batches: bool = True,
                 apply_jit: bool = False, pipeline_postproc: bool = True, custom_model_fwd=None, emb_lookup_stream: str = "data_dist",
                 embedding_lookup_after_data_dist: bool = False, **kwargs) -> None:
        super().__init__(model, optimizer, device, execute_all_batches, apply_jit, context_type=EmbeddingTrainPipelineContext,
                         pipeline_postproc=pipeline_postproc, custom_model_fwd=custom_model_fwd, **kwargs)
        self._embedding_lookup_after_data_dist = embedding_lookup_after_data_dist
        if emb_lookup_stream == "new" and device.type == "cuda":
            self._emb_lookup_stream: Optional[torch.Stream] = torch.cuda.Stream()
        elif emb_lookup_stream == "current" and device.type == "cuda":
            self._emb_lookup_stream = torch.cuda.current_stream()
        else:
            self._emb_lookup_stream = self._data_dist_stream

    def _make_forward(self, name, module, call_args, context):
        return InSyncEmbeddingPipelinedForward(name, call_args, module, context, self._emb_lookup_stream)

    def start_embedding_lookup(self, batch: Optional[In], context: EmbeddingTrainPipelineContext) -> None:
        """Run ``compute_and_output_dist`` of every pipelined module for ``batch`` ahead of its forward."""
        if batch is None or not self._pipelined:
            return
        with record_function(f"## start_embedding_lookup {context.index} ##"):
            cur = torch.get_device_module(self._device).current_stream() if self._device.type == "cuda" else None
            with self._stream_context(self._emb_lookup_stream):
                if self._emb_lookup_stream is not None and cur is not None and self._emb_lookup_stream is not cur:
                    self._emb_lookup_stream.wait_stream(cur)
                for name, module in self._pipelined_modules.items():
                    if name not in context.input_dist_tensors_requests:
                        continue
                    request = context.input_dist_tensors_requests.pop(name)
                    data = request.wait()
                    mctx = context.module_contexts[name]
                    context.embedding_a2a_requests[name] = module.compute_and_output_dist(mctx, data)

    def _step_before_forward(self) -> None:
        if self._pipelined and self.contexts[0].input_dist_tensors_requests:
            self.start_embedding_lookup(self.batches[0], cast(EmbeddingTrainPipelineContext, self.contexts[0]))


class TrainPipelineSemiSync(TrainPipelineFusedSparseDist[In, Out]):
    """Batch i+1's embedding lookup starts right after batch i's forward, i.e. before batch i's sparse
    update is applied: embeddings are one step stale from ``start_batch`` on, in exchange for overlapping
    the embedding all-to-all with the dense backward."""

    def __init__(self, model: torch.nn.Module, optimizer: torch.optim.Optimizer, device: torch.device, execute_all_batches: bool = True,
                 apply_jit: bool = False, start_batch: int = 900, stash_gradients: bool = False, pipeline_postproc: bool = True,
                 custom_model_fwd=None, strict: bool = False, **kwargs) -> None:
        super().__init__(model, optimizer, device, execute_all_batches, apply_jit, pipeline_postproc=pipeline_postproc, custom_model_fwd=custom_model_fwd, **kwargs)
        self._start_batch = start_batch
        self._stash_gradients = stash_gradients
        self._strict = strict
        self._gradients: Dict[str, torch.Tensor] = {}

    def _make_forward(self, name, module, call_args, context):
        return EmbeddingPipelinedForward(name, call_args, module, context, self._emb_lookup_stream)

    def is_semi_sync(self) -> bool:
        head = self.contexts[0].index if self.batches else None
        return head is not None and head >= self._start_batch

    def _step_before_forward(self) -> None:
        # from ``start_batch`` on the lookup of a batch was already launched one step earlier (see ``_step_after_forward``)
        self._semi = self.is_semi_sync()
        if not self._semi:
            super()._step_before_forward()

    def _step_after_forward(self) -> None:
        super()._step_after_forward()
        if self._semi and self._pipelined and len(self.batches) >= 2:
            # the stale lookup: launched before this batch's sparse update is applied
            self.start_embedding_lookup(self.batches[1], cast(EmbeddingTrainPipelineContext, self.contexts[1]))


class PrefetchTrainPipelineSparseDist(TrainPipelineSparseDist[In, Out]):
    """Adds a prefetch stage (cache pre-loading for tables kept partly outside HBM) between the input
    dist and the forward, on ``prefetch_stream``."""

    def __init__(self, model: torch.nn.Module, optimizer: torch.optim.Optimizer, device: torch.device, execute_all_batches: bool = True,
                 apply_jit: bool = False, pipeline_postproc: bool = True, custom_model_fwd=None, **kwargs) -> None:
        super().__init__(model, optimizer, device, execute_all_batches, apply_jit, context_type=PrefetchTrainPipelineContext,
                         pipeline_postproc=pipeline_postproc, custom_model_fwd=custom_model_fwd, **kwargs)
        self._prefetch_stream: Optional[torch.Stream] = torch.cuda.Stream() if device.type == "cuda" else None
        self._default_stream: Optional[torch.Stream] = torch.cuda.current_stream() if device.type == "cuda" else None

    def _make_forward(self, name, module, call_args, context):
        return PrefetchPipelinedForward(name, call_args, module, context, self._prefetch_stream)

    def _prefetch(self, batch: Optional[In], context: PrefetchTrainPipelineContext) -> None:
        if batch is None or not self._pipelined:
            return
        with record_function(f"## sharded_module_prefetch {context.index} ##"):
            with self._stream_context(self._prefetch_stream):
                if self._prefetch_stream is not None and self._data_dist_stream is not None:
                    self._prefetch_stream.wait_stream(self._data_dist_stream)
                for name, module in self._pipelined_modules.items():
                    if name not in context.input_dist_tensors_requests:
                        continue
                    data = context.input_dist_tensors_requests.pop(name).wait()
                    mctx = context.module_contexts.pop(name)
                    if hasattr(module, "prefetch"):
                        module.prefetch(ctx=mctx, dist_input=data, forward_stream=self._default_stream)
                    context.module_input_post_prefetch[name] = data
                    context.module_contexts_post_prefetch[name] = mctx

    def _step_before_forward(self) -> None:
        if self._pipelined and self.contexts[0].input_dist_tensors_requests:
            self._prefetch(self.batches[0], cast(PrefetchTrainPipelineContext, self.contexts[0]))


class EvalPipelineSparseDist(TrainPipelineSparseDist[In, Out]):
    """Forward-only pipeline; batches are loaded by a background ``DataLoadingThread``."""

    def __init__(self, model: torch.nn.Module, optimizer: torch.optim.Optimizer, device: torch.device, apply_jit: bool = False) -> None:
        super().__init__(model, optimizer, device, True, apply_jit)
        self._batch_loader: Optional[DataLoadingThread[In]] = None

    def __del__(self) -> None:
        if getattr(self, "_batch_loader", None) is not None:
            self._batch_loader.stop()

    def progress(self, dataloader_iter: Iterator[In]) -> Out:
        if self._batch_loader is None or self._batch_loader._dataloader_iter is not dataloader_iter and self._batch_loader.dataloader_iter_exhausted:
            self._batch_loader = DataLoadingThread(device=self._device, dataloader_iter=dataloader_iter, to_device_non_blocking=True, memcpy_stream=self._memcpy_stream)
            self._batch_loader.start()
        loader = self._batch_loader

        def gen():
            while True:
                b = loader.get_next_batch()
                if b is None:
                    return
                yield b

        if not hasattr(self, "_eval_iter") or self._eval_loader is not loader:
            self._eval_iter = gen()
            self._eval_loader = loader
        was_training = self._model.training
        self._model.eval()
        try:
            with torch.no_grad():
                return super().progress(self._eval_iter)
        finally:
            self._model.train(was_training)

    def copy_batch_to_gpu(self, dataloader_iter: Iterator[In]):
        # batches from the loading thread are already on the device
        context = self._create_context()
        batch = self._next_batch(dataloader_iter)
        return batch, context


class TrainPipelineSparseDistCompAutograd(TrainPipelineSparseDist[In, Out]):
    """Kept for API parity (the reference variant compiles autograd); runs the eager pipeline."""

    def __init__(self, *args, **kwargs) -> None:
        kwargs.pop("compiled_autograd_options", None)
        super().__init__(*args, **kwargs)


class StagedTrainPipeline(TrainPipeline[In, Optional[Any]]):
    """User-defined stages, each with its own stream; ``progress`` returns the batch that has passed all
    stages (the caller runs the model on it)."""

    def __init__(self, pipeline_stages: List[Any], debug_mode: bool = False, compute_stream: Optional[torch.Stream] = None,
                 on_flush_end: Optional[Callable[[], None]] = None) -> None:
        self._pipeline_stages = pipeline_stages
        self._debug_mode = debug_mode
        self._stage_outputs: List[Optional[Tuple[Any, Optional[torch.Event]]]] = [None] * len(pipeline_stages)
        self._initialized = False
        self._num_steps = 0
        self._dataloader_iter: Optional[Iterator[In]] = None
        self._dataloader_exhausted = False
        self._compute_stream = compute_stream or (torch.cuda.current_stream() if torch.cuda.is_available() else None)
        self._stream_context = torch.cuda.stream if torch.cuda.is_available() else contextlib.nullcontext
        self._flushing = False
        self.on_flush_end = on_flush_end

    @property
    def num_stages(self) -> int:
        return len(self._pipeline_stages)

    def _next_batch(self, dataloader_iter: Iterator[In]) -> Optional[In]:
        if dataloader_iter is not self._dataloader_iter:
            self._dataloader_iter = dataloader_iter
            self._dataloader_exhausted = False
        if self._dataloader_exhausted or self._flushing:
            return None
        batch = next(dataloader_iter, None)
        if batch is None:
            self._dataloader_exhausted = True
        return batch

    def _run_stage(self, stage_idx: int, item: Optional[Tuple[Any, Optional[torch.Event]]]):
        """Run stage ``stage_idx`` on ``item`` (output + completion event of the previous stage)."""
        if item is None:
            return None
        stage = self._pipeline_stages[stage_idx]
        batch, event = item
        ctx = self._stream_context(stage.stream) if stage.stream is not None else contextlib.nullcontext()
        with record_function(f"## Pipeline Stage {stage_idx} : {stage.name} ##"), ctx:
            if event is not None:
                event.wait(stage.stream) if stage.stream is not None else event.wait()
            result = stage.runnable(batch)
        new_event = None
        if stage.stream is not None and torch.cuda.is_available():
            new_event = torch.cuda.Event()
            new_event.record(stage.stream)
        return (result, new_event)

    def _shift(self, dataloader_iter: Iterator[In]) -> None:
        """One pipeline tick: every stage processes the output its predecessor produced in the last tick
        (last stage first, so stages of different batches overlap on their streams)."""
        for i in range(self.num_stages - 1, 0, -1):
            self._stage_outputs[i] = self._run_stage(i, self._stage_outputs[i - 1])
        nb = self._next_batch(dataloader_iter)
        self._stage_outputs[0] = self._run_stage(0, (nb, None)) if nb is not None else None

    def set_flush(self, flush: bool) -> None:
        self._flushing = flush

    def progress(self, dataloader_iter: Iterator[In]) -> Optional[Any]:
        if not self._initialized:
            for _ in range(self.num_stages):
                self._shift(dataloader_iter)
            self._initialized = True
        out = self._stage_outputs[-1]
        self._num_steps += 1
        self._shift(dataloader_iter)
        if out is None:
            if self._flushing and all(o is None for o in self._stage_outputs):
                self._flushing = False
                if self.on_flush_end is not None:
                    self.on_flush_end()
                return self.progress(dataloader_iter)
            if any(o is not None for o in self._stage_outputs):
                return self.progress(dataloader_iter)
            return None
        result, event = out
        if event is not None and self._compute_stream is not None:
            event.wait(self._compute_stream)
        if result is not None and self._compute_stream is not None and hasattr(result, "record_stream"):
            result.record_stream(self._compute_stream)
        return result
