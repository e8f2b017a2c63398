"""Pipeline plumbing: device copies, stream hand-off, discovery of pipelined modules and of the
batch fields they consume, starting the sparse data dist, a background data-loading thread.

The reference finds each sharded module's inputs by fx-tracing the model
(``torchrec/distributed/train_pipeline/utils.py:287-420``).  Here the first batch runs through the
model unpipelined while a pre-forward hook records which object each sharded module received; that
object is then located inside the batch (attributes / items, by identity) and the resulting accessor
path (``ArgInfo``) is used for every later batch.  Models need not be fx-traceable.
"""
from __future__ import annotations

import dataclasses
import logging
import queue
import threading
from typing import Any, Callable, Dict, Generic, Iterator, List, Optional, Set, Tuple, Type, TypeVar, cast

import torch
from torch.autograd.profiler import record_function

from torchrec_b200.distributed.embedding_sharding import FusedKJTListSplitsAwaitable, KJTListSplitsAwaitable
from torchrec_b200.distributed.train_pipeline.pipeline_context import TrainPipelineContext
from torchrec_b200.distributed.train_pipeline.types import ArgInfo, CallArgs
from torchrec_b200.distributed.types import Awaitable, ShardedModule
from torchrec_b200.streamable import Multistreamable, Pipelineable

logger: logging.Logger = logging.getLogger(__name__)

In = TypeVar("In", bound=Pipelineable)
Out = TypeVar("Out")
StageOut = TypeVar("StageOut")
RunnableType = Callable[..., StageOut]
StageOutputWithEvent = Tuple[Optional[StageOut], Optional[torch.Event]]


def _to_device(batch: In, device: torch.device, non_blocking: bool) -> In:
    assert isinstance(batch, (torch.Tensor, Pipelineable)), f"{type(batch)} must implement Pipelineable interface"
    return cast(In, batch.to(device=device, non_blocking=non_blocking))


def get_h2d_func(batch: In, device: torch.device) -> Pipelineable:
    """The default host-to-device step of a data-loading stage: ``batch.to(device, non_blocking=True)``."""
    return batch.to(device, non_blocking=True)


def _wait_for_batch(batch: In, stream: Optional[torch.Stream]) -> None:
    """Make the current stream wait for ``stream`` and mark ``batch`` as used on the current stream."""
    if stream is None:
        return
    device = stream.device
    torch.get_device_module(device).current_stream().wait_stream(stream)
    cur_stream = torch.get_device_module(device).current_stream()
    assert isinstance(batch, (torch.Tensor, Multistreamable)), f"{type(batch)} must implement Multistreamable interface"
    batch.record_stream(cur_stream)


def _wait_for_events(batch: In, context: TrainPipelineContext, stream: Optional[torch.Stream]) -> None:
    if stream is None:
        return
    assert context.event is not None
    context.event.wait()
    context.event = None
    cur_stream = torch.get_device_module(stream.device).current_stream()
    batch.record_stream(cur_stream)


# ---- discovery of pipelined modules and their inputs --------------------------------------------------
def find_sharded_modules(model: torch.nn.Module) -> Dict[str, ShardedModule]:
    """Sharded modules by qualified name (DDP / DMP wrapper names are kept: they are only used as keys)."""
    out: Dict[str, ShardedModule] = {}
    for name, m in model.named_modules():
        if isinstance(m, ShardedModule):
            out[name] = m
    return out


def _find_path(root: Any, target: Any, max_depth: int = 4) -> Optional[ArgInfo]:
    """Locate ``target`` (by identity) inside ``root`` following attributes and items."""
    seen: Set[int] = set()

    def rec(obj: Any, attrs: List[Any], getitems: List[bool], depth: int) -> Optional[ArgInfo]:
        if obj is target:
            return ArgInfo(list(attrs), list(getitems))
        if depth >= max_depth or id(obj) in seen:
            return None
        seen.add(id(obj))
        children: List[Tuple[Any, bool, Any]] = []
        if isinstance(obj, dict):
            children = [(k, True, v) for k, v in obj.items()]
        elif isinstance(obj, (list, tuple)):
            children = [(i, True, v) for i, v in enumerate(obj)]
        elif dataclasses.is_dataclass(obj) and not isinstance(obj, type):
            children = [(f.name, False, getattr(obj, f.name)) for f in dataclasses.fields(obj)]
        elif hasattr(obj, "__dict__") and not isinstance(obj, (torch.Tensor, torch.nn.Module)):
            children = [(k, False, v) for k, v in vars(obj).items() if not k.startswith("__")]
        for key, is_item, child in children:
            if isinstance(child, (int, float, str, bool, type(None))):
                continue
            r = rec(child, attrs + [key], getitems + [is_item], depth + 1)
            if r is not None:
                return r
        return None

    return rec(root, [], [], 0)


def find_postproc_candidates(model: torch.nn.Module, sharded: Dict[str, ShardedModule]) -> Dict[str, torch.nn.Module]:
    """Modules that may run ahead of the model forward as input post-processing: not the root, not a sharded module nor inside
    one, not a container of one, and without trainable parameters (running a trained module a batch early would read stale
    weights)."""
    out: Dict[str, torch.nn.Module] = {}
    sharded_names = list(sharded.keys())
    for name, m in model.named_modules():
        if name == "" or isinstance(m, ShardedModule):
            continue
        if any(s == name or s.startswith(name + ".") or name.startswith(s + ".") for s in sharded_names):
            continue
        if any(p.requires_grad for p in m.parameters()):
            continue
        out[name] = m
    return out


class ArgRecorder:
    """Hooks that remember the first call of every sharded module (its arguments) and, when post-processing modules are to be
    pipelined too, of every candidate post-processing module (arguments and output)."""

    def __init__(self, modules: Dict[str, ShardedModule], postproc_candidates: Optional[Dict[str, torch.nn.Module]] = None) -> None:
        self.calls: Dict[str, Tuple[Tuple[Any, ...], Dict[str, Any]]] = {}
        self.postproc_calls: Dict[str, Tuple[Tuple[Any, ...], Dict[str, Any], Any]] = {}
        self.postproc_modules: Dict[str, torch.nn.Module] = dict(postproc_candidates or {})
        self.postprocs: Dict[str, Any] = {}  # fqn -> PipelinedPostproc, filled by resolve()
        self._handles = []
        for name, m in modules.items():
            self._handles.append(m.register_forward_pre_hook(self._make_hook(name), with_kwargs=True))
        for name, m in self.postproc_modules.items():
            self._handles.append(m.register_forward_hook(self._make_postproc_hook(name), with_kwargs=True))

    def _make_hook(self, name: str):
        def hook(module, args, kwargs):
            if name not in self.calls:
                self.calls[name] = (args, dict(kwargs))
            return None

        return hook

    def _make_postproc_hook(self, name: str):
        def hook(module, args, kwargs, output):
            if name not in self.postproc_calls:
                self.postproc_calls[name] = (args, dict(kwargs), output)
            return None

        return hook

    def remove(self) -> None:
        for h in self._handles:
            h.remove()
        self._handles = []

    def _locate(self, batch: Any, value: Any, depth: int = 0) -> Optional[ArgInfo]:
        """Where ``value`` comes from: a literal, the batch, or the output of a post-processing module whose own inputs can be
        located the same way."""
        if isinstance(value, (int, float, str, bool, type(None))):
            return ArgInfo(constant=(value,))
        found = _find_path(batch, value)
        if found is not None or depth > 4:
            return found
        from torchrec_b200.distributed.train_pipeline.postproc import PipelinedPostproc

        for name, (args, kwargs, output) in self.postproc_calls.items():
            inside = _find_path(output, value)
            if inside is None:
                continue
            pp = self.postprocs.get(name)
            if pp is None:
                call = self._locate_all(batch, args, kwargs, depth + 1)
                if call is None:
                    continue
                pp = PipelinedPostproc(self.postproc_modules[name], name, call)
                self.postprocs[name] = pp
            inside.postproc = pp
            return inside
        return None

    def _locate_all(self, batch: Any, args: Tuple[Any, ...], kwargs: Dict[str, Any], depth: int = 0) -> Optional[CallArgs]:
        ca = CallArgs()
        for a in args:
            p = self._locate(batch, a, depth)
            if p is None:
                return None
            ca.args.append(p)
        for k, a in kwargs.items():
            p = self._locate(batch, a, depth)
            if p is None:
                return None
            ca.kwargs[k] = p
        return ca

    def resolve(self, batch: Any) -> Dict[str, CallArgs]:
        """Accessor paths for every recorded sharded module whose arguments all come from the batch, directly or through
        post-processing modules."""
        out: Dict[str, CallArgs] = {}
        for name, (args, kwargs) in self.calls.items():
            ca = self._locate_all(batch, args, kwargs)
            if ca is not None:
                out[name] = ca
            else:
                logger.warning(f"train pipeline: inputs of sharded module '{name}' are computed inside the model; it will not be pipelined")
        return out


# ---- starting / finishing the sparse data dist ------------------------------------------------------------
def _start_data_dist(pipelined_modules: Dict[str, ShardedModule], call_args: Dict[str, CallArgs], batch: Pipelineable,
                     context: TrainPipelineContext) -> None:
    """Stage 1 of every pipelined module's input dist for ``batch`` (call on the data-dist stream)."""
    if context.version == 0:
        context.input_dist_splits_requests.clear()
        context.module_contexts_next_batch.clear()
        context.fused_splits_awaitables.clear()
    for name, module in pipelined_modules.items():
        ca = call_args.get(name)
        if ca is None:
            continue
        args, kwargs = ca.build_args_kwargs(batch, context)
        module_ctx = module.create_context()
        if context.version == 0:
            context.module_contexts_next_batch[name] = module_ctx
        else:
            context.module_contexts[name] = module_ctx
        context.input_dist_splits_requests[name] = module.input_dist(module_ctx, *args, **kwargs)
    _fuse_input_dist_splits(context)


def _fuse_input_dist_splits(context: TrainPipelineContext) -> None:
    """Group the stage-1 requests by process group and exchange all their split sizes in one collective each."""
    names_per_pg: Dict[Any, List[str]] = {}
    for name, request in context.input_dist_splits_requests.items():
        pg = None
        if isinstance(request, KJTListSplitsAwaitable):
            for aw in request.awaitables:
                if hasattr(aw, "_pg"):
                    pg = aw._pg
                    break
            names_per_pg.setdefault(pg, []).append(name)
    for pg, names in names_per_pg.items():
        ctxs = context.module_contexts_next_batch if context.version == 0 else context.module_contexts
        context.fused_splits_awaitables.append(
            (
                names,
                FusedKJTListSplitsAwaitable(
                    requests=[context.input_dist_splits_requests[n] for n in names],
                    contexts=[ctxs[n] for n in names], pg=pg,
                ),
            )
        )


def _wait_data_dist(context: TrainPipelineContext) -> None:
    """Finish stage 1 (split sizes are now known) and launch stage 2 (payload all-to-alls)."""
    for names, awaitable in context.fused_splits_awaitables:
        for name, request in zip(names, awaitable.wait()):
            context.input_dist_tensors_requests[name] = request
    fused = {n for names, _ in context.fused_splits_awaitables for n in names}
    for name, request in context.input_dist_splits_requests.items():
        if name not in fused:
            # a module whose input distribution has no split-size stage (the fused sparse engine keeps sizes on the device)
            context.input_dist_tensors_requests[name] = request.wait()
    context.input_dist_splits_requests.clear()
    context.fused_splits_awaitables.clear()


class DataLoadingThread(threading.Thread, Generic[In]):
    """Background thread that pulls batches from the iterator and copies them to the device on
    ``memcpy_stream`` so that ``get_next_batch`` rarely blocks."""

    def __init__(self, device: torch.device, dataloader_iter: Iterator[In], to_device_non_blocking: bool,
                 memcpy_stream_priority: int = 0, memcpy_stream: Optional[torch.Stream] = None) -> None:
        super().__init__(name="DataLoadingThread", daemon=True)
        self._stop: bool = False
        self.dataloader_iter_exhausted: bool = False
        self._dataloader_iter = dataloader_iter
        self._buffer_empty_event = threading.Event()
        self._buffer_filled_event = threading.Event()
        if memcpy_stream is None:
            self._memcpy_stream: Optional[torch.Stream] = (
                torch.get_device_module(device).Stream(priority=memcpy_stream_priority) if device.type in ["cuda", "mtia"] else None
            )
        else:
            self._memcpy_stream = memcpy_stream
        self._device = device
        self._to_device_non_blocking = to_device_non_blocking
        self._buffered: Optional[In] = None
        self._buffer_empty_event.set()

    def run(self) -> None:
        if self._device.type == "cuda" and torch.cuda.is_available():
            torch.cuda.set_device(self._device)
        while not self._stop:
            self._buffer_empty_event.wait()
            if self._stop:
                self._buffer_filled_event.set()
                return
            with record_function("## load_batch ##"):
                try:
                    batch = next(self._dataloader_iter)
                except StopIteration:
                    self.dataloader_iter_exhausted = True
                    self._buffer_filled_event.set()
                    return
            with record_function("## copy_batch_to_gpu ##"):
                if self._memcpy_stream is not None:
                    with torch.get_device_module(self._device).stream(self._memcpy_stream):
                        self._buffered = _to_device(batch, self._device, self._to_device_non_blocking)
                else:
                    self._buffered = _to_device(batch, self._device, self._to_device_non_blocking)
                self._buffer_empty_event.clear()
                self._buffer_filled_event.set()

    def stop(self) -> None:
        logger.info("Stopping data loading thread...")
        self._stop = True
        self._buffer_filled_event.set()
        self._buffer_empty_event.set()

    def get_next_batch(self, none_throws: bool = False) -> Optional[In]:
        """Next batch, already on the device; ``None`` (or ``StopIteration``) at the end of the data."""
        self._buffer_filled_event.wait()
        batch = self._buffered
        if batch is None:
            if none_throws:
                raise StopIteration
            return None
        self._buffered = None
        self._buffer_filled_event.clear()
        self._buffer_empty_event.set()
        return batch


def use_context_for_postprocs(module: torch.nn.Module, context: TrainPipelineContext) -> None:
    """Point every pipelined post-processing module at the context of the batch whose forward is about to run."""
    from torchrec_b200.distributed.train_pipeline.postproc import PipelinedPostproc

    for m in module.modules():
        if isinstance(m, PipelinedPostproc):
            m.set_context(context)
