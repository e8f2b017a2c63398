"""``TrainPipelineGraphed``: the whole training step -- sparse input distribution, embedding lookup, dense forward, loss,
backward, fused embedding update, dense gradient averaging, dense optimizer -- captured ONCE as a CUDA graph and replayed.

Why: on a B200 the device needs a few milliseconds for a step whose launches cost the host about as long to issue; a
replayed graph costs the host tens of microseconds, so the step time is the device time.  It is the B200-native stand-in
for the reference's compiled pipeline (``TrainPipelinePT2``, ``torchrec/distributed/train_pipeline/train_pipelines.py:340``).

What makes the step capturable (all provided by this package):

* the fused sparse engine keeps every size on the device (``distributed/fused_sparse_engine.py``);
* dense gradients are averaged by a peer-memory kernel (``distributed/peer_data_parallel.py``), not by host-driven buckets;
* the dense optimizer is one launch with device-side step counters (``optim/fused_dense.py``).

Batches are copied into *static* input tensors (host batches land in one of two staging sets on a copy stream while the
previous replay runs).  Id tensors are padded to a capacity, so batches with different numbers of ids share one graph;
a batch that exceeds the capacity, or has another batch size, is run eagerly (and counted in ``eager_steps``).

The first ``warmup_steps`` steps run eagerly (they also size the engine's receive buffers), then the step is captured.
Outputs are the model's outputs as *static* tensors: read or clone them before the next ``progress`` call.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Callable, Dict, Iterator, List, Optional, Tuple

import torch

from torchrec_b200.distributed.peer_memory import poll_all
from torchrec_b200.distributed.train_pipeline.train_pipelines import TrainPipeline
from torchrec_b200.distributed.train_pipeline.utils import In, Out
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

_ID_SLACK = 1.25


def _walk(obj: Any, fn: Callable[[str, Any], Any], path: str = "") -> Any:
    """Rebuild ``obj`` with every tensor leaf replaced by ``fn(kind, leaf)``; kind is "ids" for the values / weights of a
    KeyedJaggedTensor (variable length) and "t" otherwise."""
    if isinstance(obj, torch.Tensor):
        return fn("t", obj)
    if isinstance(obj, KeyedJaggedTensor):
        lengths = obj.lengths()
        return KeyedJaggedTensor(
            keys=obj.keys(), values=fn("ids", obj.values()), weights=None if obj.weights_or_none() is None else fn("ids", obj.weights()),
            lengths=fn("t", lengths), stride=obj.stride(),
        )
    if dataclasses.is_dataclass(obj) and not isinstance(obj, type):
        return dataclasses.replace(obj, **{f.name: _walk(getattr(obj, f.name), fn, path + "." + f.name) for f in dataclasses.fields(obj)})
    if isinstance(obj, dict):
        return {k: _walk(v, fn, path) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_walk(v, fn, path) for v in obj)
    return obj


def _leaves(obj: Any) -> List[Tuple[str, torch.Tensor]]:
    out: List[Tuple[str, torch.Tensor]] = []
    _walk(obj, lambda kind, t: (out.append((kind, t)), t)[1])
    return out


class TrainPipelineGraphed(TrainPipeline[In, Out]):
    def __init__(self, model: torch.nn.Module, optimizer: torch.optim.Optimizer, device: torch.device, warmup_steps: int = 3,
                 custom_model_fwd: Optional[Callable[[In], Tuple[torch.Tensor, Out]]] = None, train: bool = True) -> None:
        assert device.type == "cuda", "CUDA graphs need a CUDA device"
        self._model, self._optimizer, self._device = model, optimizer, device
        self._fwd = custom_model_fwd if custom_model_fwd is not None else model
        self._warmup = max(int(warmup_steps), 1)
        self._train = train
        self._steps = 0
        self.eager_steps = 0
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self._static_batch: Any = None
        self._static_leaves: List[Tuple[str, torch.Tensor]] = []
        self._static_out: Any = None
        self._sig: Optional[Tuple[Any, ...]] = None
        self._copy_stream = torch.cuda.Stream(device=device)
        self._landing: List[Optional[List[torch.Tensor]]] = [None, None]
        self._landed_event: List[Optional[torch.cuda.Event]] = [None, None]
        self._consumed_event: List[Optional[torch.cuda.Event]] = [None, None]
        self._next: Optional[Tuple[int, Any, List[Tuple[str, torch.Tensor]]]] = None
        self._k = 0
        self._exhausted = False
        self._pad_ids = False

    # ---- one step, eagerly ------------------------------------------------------------------------------------------
    def _step(self, batch: Any) -> Any:
        if self._train:
            self._optimizer.zero_grad()
            losses, output = self._fwd(batch)
            torch.sum(losses, dim=0).backward()
            self._optimizer.step()
            return output
        with torch.no_grad():
            return self._fwd(batch)[1]

    # ---- static inputs --------------------------------------------------------------------------------------------------
    def _signature(self, leaves: List[Tuple[str, torch.Tensor]]) -> Tuple[Any, ...]:
        return tuple((kind, t.dtype, tuple(t.shape) if (kind == "t" or not self._pad_ids) else None) for kind, t in leaves)

    def _fits(self, leaves: List[Tuple[str, torch.Tensor]]) -> bool:
        if self._sig is None or self._signature(leaves) != self._sig:
            return False
        return all(kind == "t" or t.numel() <= s.numel() for (kind, t), (_, s) in zip(leaves, self._static_leaves))

    def _make_static(self, batch: Any) -> None:
        def alloc(kind: str, t: torch.Tensor) -> torch.Tensor:
            n = t.numel() if (kind == "t" or not self._pad_ids) else max(int(t.numel() * _ID_SLACK) + 1024, 1024)
            s = torch.zeros((n,) if kind == "ids" else tuple(t.shape), dtype=t.dtype, device=self._device)
            return s

        self._static_batch = _walk(batch, alloc)
        self._static_leaves = _leaves(self._static_batch)
        self._sig = self._signature(_leaves(batch))
        self._landing = [[torch.empty_like(s) for _, s in self._static_leaves] for _ in range(2)]

    # ---- feeding ---------------------------------------------------------------------------------------------------------
    def _start_copy(self, dataloader_iter: Iterator[In]) -> None:
        """Fetch the next batch and start moving it towards the device on the copy stream."""
        if self._exhausted:
            self._next = None
            return
        try:
            batch = next(dataloader_iter)
        except StopIteration:
            self._exhausted = True
            self._next = None
            return
        leaves = _leaves(batch)
        k = self._k
        self._k ^= 1
        if self._graph is not None and self._fits(leaves):
            land = self._landing[k]
            with torch.cuda.stream(self._copy_stream):
                if self._consumed_event[k] is not None:
                    self._copy_stream.wait_event(self._consumed_event[k])
                for (kind, t), dst in zip(leaves, land):
                    dst.view(-1)[: t.numel()].copy_(t.reshape(-1), non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self._copy_stream)
            self._landed_event[k] = ev
            self._next = (k, None, leaves)
        else:
            with torch.cuda.stream(self._copy_stream):
                dev_batch = batch.to(self._device, non_blocking=True) if hasattr(batch, "to") else batch
                ev = torch.cuda.Event()
                ev.record(self._copy_stream)
            self._landed_event[k] = ev
            self._next = (k, dev_batch, leaves)

    def progress(self, dataloader_iter: Iterator[In]) -> Out:
        if self._next is None and not self._exhausted:
            self._start_copy(dataloader_iter)
        if self._next is None:
            raise StopIteration
        k, dev_batch, leaves = self._next
        cur = torch.cuda.current_stream()
        cur.wait_event(self._landed_event[k])
        if dev_batch is None:
            # the batch sits in landing set k: move it into the graph's inputs, replay
            for (_, s), src in zip(self._static_leaves, self._landing[k]):
                s.copy_(src, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(cur)
            self._consumed_event[k] = ev
            self._start_copy(dataloader_iter)
            self._graph.replay()
            self._steps += 1
            poll_all()  # a bounded device wait that ran out in an earlier step raises here
            return self._static_out
        for _, t in _leaves(dev_batch):
            t.record_stream(cur)
        self._start_copy(dataloader_iter)
        if self._graph is None and self._steps + 1 >= self._warmup:
            out = self._capture(dev_batch)
            self._steps += 1
            return out
        out = self._step(dev_batch)
        self._steps += 1
        if self._graph is not None:
            self.eager_steps += 1
        return out

    # ---- capture -----------------------------------------------------------------------------------------------------------
    def _can_pad_ids(self) -> bool:
        """Ids may be padded to a capacity only when every sharded module reads them through offsets, i.e. runs on the fused
        sparse engine (its backward skips padding through a device-side count)."""
        from torchrec_b200.distributed.types import ShardedModule

        found = False
        for m in self._model.modules():
            if isinstance(m, ShardedModule):
                found = True
                if getattr(m, "_engine", None) is None:
                    return False
        return found

    def _capture(self, example: Any) -> Any:
        """Train on ``example`` through the static inputs (eagerly: this is the batch's real step and it builds every lazily
        created cache at its final address), then record the same step into a graph without running it."""
        self._pad_ids = self._can_pad_ids()
        self._make_static(example)
        for (kind, t), (_, s) in zip(_leaves(example), self._static_leaves):
            s.view(-1)[: t.numel()].copy_(t.reshape(-1))
        out = self._step(self._static_batch)
        torch.cuda.synchronize(self._device)
        self._static_batch = _walk(self._static_batch, lambda kind, t: t)  # fresh containers: no cached derived tensors
        self._static_leaves = _leaves(self._static_batch)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self._static_out = self._step(self._static_batch)
        self._graph = graph
        return out

    @property
    def captured(self) -> bool:
        return self._graph is not None
