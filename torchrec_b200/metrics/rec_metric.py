"""Metric framework: windowed + lifetime states, per-task or fused-task computations, cross-rank sync.

A ``RecMetricComputation`` owns named state tensors with a leading ``n_tasks`` dim.  Every state exists
twice: the *lifetime* value (sum/max/cat over all updates) and, optionally, a *window* value over the
last ``window_size`` examples, kept as a running aggregate plus a queue of per-update contributions so
that the oldest updates can be subtracted when the window overflows.  ``compute()`` first combines the
states of all ranks (all-reduce for sum/max states, all-gather for list states), then evaluates the
metric from them, so every reported value is a global one.

``RecMetric`` fans a ``{task: tensor}`` update out to its computations (one per task, or one fused over
all tasks), buffers updates when ``fused_update_limit > 1`` and names the results.

Counterpart of ``torchrec/metrics/rec_metric.py`` (``RecMetricComputation`` ``:108``, ``RecMetric``
``:279``, ``RecMetricList`` ``:871``); built on ``nn.Module`` buffers instead of an external metrics package.
"""
from __future__ import annotations

import abc
import math
from collections import deque
from dataclasses import dataclass
from typing import Any, Callable, Deque, Dict, Iterator, List, Optional, Tuple, Type, Union

import torch
import torch.distributed as dist
from torch import nn

from torchrec_b200.metrics.metrics_config import BatchSizeStage, RecComputeMode, RecTaskInfo
from torchrec_b200.metrics.metrics_namespace import MetricNameBase, MetricNamespaceBase, MetricPrefix, compose_metric_key

RecModelOutput = Union[torch.Tensor, Dict[str, torch.Tensor]]


class RecMetricException(Exception):
    pass


@dataclass(frozen=True)
class MetricComputationReport:
    name: MetricNameBase
    metric_prefix: MetricPrefix
    value: torch.Tensor
    description: Optional[str] = None


DefaultValueT = Union[torch.Tensor, List[torch.Tensor]]
ReduceT = Union[str, Callable[[torch.Tensor], torch.Tensor]]


class WindowBuffer:
    """Queue of per-update contributions of one windowed state with the number of examples of each."""

    def __init__(self, max_size: int, max_buffer_count: int) -> None:
        self._max_size = max_size
        self._max_buffer_count = max_buffer_count
        self._buffers: Deque[torch.Tensor] = deque(maxlen=max_buffer_count)
        self._used_sizes: Deque[int] = deque(maxlen=max_buffer_count)
        self._window_used_size = 0

    def aggregate_state(self, window_state: torch.Tensor, curr_state: torch.Tensor, size: int) -> None:
        """Add ``curr_state`` (from ``size`` examples) to ``window_state`` in place and drop what fell out."""

        def remove(window_state: torch.Tensor) -> None:
            window_state -= self._buffers.popleft()
            self._window_used_size -= self._used_sizes.popleft()

        if len(self._buffers) == self._buffers.maxlen:
            remove(window_state)
        self._buffers.append(curr_state)
        self._used_sizes.append(size)
        window_state += curr_state
        self._window_used_size += size
        while self._window_used_size > self._max_size:
            remove(window_state)

    @property
    def buffers(self) -> Deque[torch.Tensor]:
        return self._buffers


class RecMetricComputation(nn.Module, abc.ABC):
    """States + math of one metric for ``n_tasks`` tasks.  Subclasses call ``_add_state`` in ``__init__`` and
    implement ``update`` and ``_compute``."""

    _batch_window_buffers: Optional[Dict[str, WindowBuffer]]

    def __init__(self, my_rank: int, batch_size: int, n_tasks: int, window_size: int, compute_on_all_ranks: bool = False,
                 should_validate_update: bool = False, fuse_state_tensors: bool = False,
                 process_group: Optional[dist.ProcessGroup] = None, fused_update_limit: int = 0, allow_missing_label_with_zero_weight: bool = False,
                 *args: Any, **kwargs: Any) -> None:
        super().__init__()
        self._my_rank = my_rank
        self._n_tasks = n_tasks
        self._batch_size = batch_size
        self._window_size = window_size
        self._compute_on_all_ranks = compute_on_all_ranks
        self._should_validate_update = should_validate_update
        self._fuse_state_tensors = fuse_state_tensors
        self._process_group = process_group
        self._state_names: List[str] = []
        self._reductions: Dict[str, ReduceT] = {}
        self._defaults: Dict[str, DefaultValueT] = {}
        self._persistent: Dict[str, bool] = {}
        self._list_states: Dict[str, List[torch.Tensor]] = {}
        if window_size > 0:
            self._batch_window_buffers = {}
        else:
            self._batch_window_buffers = None
        if compute_on_all_ranks:
            self._register_load_state_dict_pre_hook(lambda *a, **k: None)

    # ---- states -------------------------------------------------------------------------------------
    @staticmethod
    def get_window_state_name(state_name: str) -> str:
        return f"window_{state_name}"

    def get_window_state(self, state_name: str) -> torch.Tensor:
        return getattr(self, self.get_window_state_name(state_name))

    def _add_state(self, name: str, default: DefaultValueT, add_window_state: bool, dist_reduce_fx: ReduceT = "sum",
                   persistent: bool = True, **kwargs: Any) -> None:
        """Register lifetime state ``name`` (tensor buffer, or python list of tensors when ``default`` is a list) and,
        if asked and a window is configured, its windowed twin ``window_<name>``."""
        self._state_names.append(name)
        self._reductions[name] = dist_reduce_fx
        self._defaults[name] = default if isinstance(default, list) else default.detach().clone()
        self._persistent[name] = persistent
        if isinstance(default, list):
            self._list_states[name] = [t.detach().clone() for t in default]
        else:
            self.register_buffer(name, default.detach().clone(), persistent=persistent)
        if add_window_state:
            if self._batch_window_buffers is None:
                raise RuntimeError("Users is adding a window state while window metric is disabled.")
            assert not isinstance(default, list), "window states must be tensors"
            wname = self.get_window_state_name(name)
            self._state_names.append(wname)
            self._reductions[wname] = dist_reduce_fx
            self._defaults[wname] = default.detach().clone()
            self._persistent[wname] = persistent
            self.register_buffer(wname, default.detach().clone(), persistent=persistent)
            self._batch_window_buffers[wname] = WindowBuffer(
                max_size=self._window_size, max_buffer_count=max(1, math.ceil(self._window_size / max(self._batch_size, 1)))
            )

    def _aggregate_window_state(self, state_name: str, state: torch.Tensor, num_samples: int) -> None:
        if self._batch_window_buffers is None:
            raise RuntimeError(f"Users is adding a window state while window metric is disabled.")
        wname = self.get_window_state_name(state_name)
        assert self._batch_window_buffers is not None
        self._batch_window_buffers[wname].aggregate_state(getattr(self, wname), curr_state=state, size=num_samples)

    def __getattr__(self, name: str) -> Any:
        ls = self.__dict__.get("_list_states")
        if ls is not None and name in ls:
            return ls[name]
        return super().__getattr__(name)

    def reset(self) -> None:
        for name in self._state_names:
            default = self._defaults[name]
            if isinstance(default, list):
                self._list_states[name] = [t.detach().clone().to(t.device) for t in default]
            else:
                getattr(self, name).copy_(default.to(getattr(self, name).device))
        if self._batch_window_buffers is not None:
            for wname, buf in list(self._batch_window_buffers.items()):
                self._batch_window_buffers[wname] = WindowBuffer(buf._max_size, buf._max_buffer_count)

    # ---- update / compute ---------------------------------------------------------------------------
    @abc.abstractmethod
    def update(self, *, predictions: Optional[torch.Tensor], labels: torch.Tensor, weights: Optional[torch.Tensor], **kwargs: Any) -> None:
        ...

    @abc.abstractmethod
    def _compute(self) -> List[MetricComputationReport]:
        ...

    def pre_compute(self) -> None:
        """Hook that runs before the cross-rank sync of ``compute`` (e.g. flush buffered updates)."""

    def _sync_and_compute(self) -> List[MetricComputationReport]:
        """Replace local states by their global combination for the duration of ``_compute``."""
        pg = self._process_group
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(pg) == 1:
            return self._compute()
        saved: Dict[str, Any] = {}
        world = dist.get_world_size(pg)
        for name in self._state_names:
            red = self._reductions[name]
            if name in self._list_states:
                local = self._list_states[name]
                saved[name] = local
                gathered: List[torch.Tensor] = []
                for t in local:
                    # ranks may hold different lengths on the last dim: exchange sizes, pad, trim
                    n = torch.tensor([t.shape[-1]], device=t.device, dtype=torch.int64)
                    sizes = [torch.zeros_like(n) for _ in range(world)]
                    dist.all_gather(sizes, n, group=pg)
                    m = int(max(int(s) for s in sizes))
                    pad = t.new_zeros(t.shape[:-1] + (m,))
                    pad[..., : t.shape[-1]] = t
                    outs = [torch.empty_like(pad) for _ in range(world)]
                    dist.all_gather(outs, pad, group=pg)
                    gathered.append(torch.cat([o[..., : int(s)] for o, s in zip(outs, sizes)], dim=-1))
                self._list_states[name] = gathered
                continue
            buf = getattr(self, name)
            saved[name] = buf.detach().clone()
            if red == "sum":
                dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=pg)
            elif red == "max":
                dist.all_reduce(buf, op=dist.ReduceOp.MAX, group=pg)
            elif red == "min":
                dist.all_reduce(buf, op=dist.ReduceOp.MIN, group=pg)
            elif red == "mean":
                dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=pg)
                buf /= world
            elif callable(red):
                outs = [torch.empty_like(buf) for _ in range(world)]
                dist.all_gather(outs, buf, group=pg)
                buf.copy_(red(torch.stack(outs)))
            elif red is None or red == "none":
                pass
            else:
                raise ValueError(f"unknown reduction {red!r} for state {name}")
        try:
            return self._compute()
        finally:
            for name, v in saved.items():
                if name in self._list_states:
                    self._list_states[name] = v
                else:
                    getattr(self, name).copy_(v)

    def compute(self) -> List[MetricComputationReport]:
        self.pre_compute()
        with torch.no_grad():
            if self._my_rank == 0 or self._compute_on_all_ranks or (dist.is_available() and dist.is_initialized()):
                return self._sync_and_compute()
        return []

    def local_compute(self) -> List[MetricComputationReport]:
        with torch.no_grad():
            return self._compute()

    # list states are not buffers: carry them through state_dict explicitly
    def get_extra_state(self) -> Dict[str, List[torch.Tensor]]:
        return {k: [t.cpu() for t in v] for k, v in self._list_states.items() if self._persistent.get(k, True)}

    def set_extra_state(self, state: Dict[str, List[torch.Tensor]]) -> None:
        for k, v in (state or {}).items():
            if k in self._list_states:
                dev = self._list_states[k][0].device if self._list_states[k] else torch.device("cpu")
                self._list_states[k] = [t.to(dev) for t in v]


class RecMetric(nn.Module, abc.ABC):
    """One metric over a list of tasks.  Subclasses set ``_namespace`` and ``_computation_class``.

    ``update`` takes ``{task name: tensor}`` dicts (or, in the fused modes, already stacked ``[n_tasks, B]``
    tensors); ``compute`` returns ``{"<namespace>-<task>|<prefix><name>": value}``.
    """

    _computation_class: Type[RecMetricComputation]
    _namespace: MetricNamespaceBase
    LABELS: str = "labels"
    PREDICTIONS: str = "predictions"
    WEIGHTS: str = "weights"

    def __init__(self, world_size: int, my_rank: int, batch_size: int, tasks: List[RecTaskInfo],
                 compute_mode: RecComputeMode = RecComputeMode.UNFUSED_TASKS_COMPUTATION, window_size: int = 100,
                 fused_update_limit: int = 0, compute_on_all_ranks: bool = False, should_validate_update: bool = False,
                 process_group: Optional[dist.ProcessGroup] = None, batch_size_stages: Optional[List[BatchSizeStage]] = None,
                 **kwargs: Any) -> None:
        torch._C._log_api_usage_once(f"torchrec_b200.metrics.rec_metric.{self.__class__.__name__}")
        if compute_mode in (RecComputeMode.FUSED_TASKS_COMPUTATION, RecComputeMode.FUSED_TASKS_AND_STATES_COMPUTATION) and fused_update_limit > 0:
            raise ValueError("The fused tasks computation and the fused update cannot be set at the same time")
        super().__init__()
        self._world_size = world_size
        self._my_rank = my_rank
        self._window_size = math.ceil(window_size / world_size)   # window is global, every rank keeps its share
        self._batch_size = batch_size
        self._batch_size_stages = batch_size_stages
        self._tasks = tasks
        self._compute_mode = compute_mode
        self._fused_update_limit = fused_update_limit
        self._should_validate_update = should_validate_update
        self._default_weights: Dict[Tuple[int, ...], torch.Tensor] = {}
        self._required_inputs: set = set()
        self._update_buffers: Dict[str, List[RecModelOutput]] = {self.PREDICTIONS: [], self.LABELS: [], self.WEIGHTS: []}
        self._kwargs = kwargs
        fuse_states = compute_mode == RecComputeMode.FUSED_TASKS_AND_STATES_COMPUTATION
        common = dict(my_rank=my_rank, batch_size=batch_size, window_size=self._window_size, compute_on_all_ranks=compute_on_all_ranks,
                      should_validate_update=should_validate_update, process_group=process_group)
        if compute_mode in (RecComputeMode.FUSED_TASKS_COMPUTATION, RecComputeMode.FUSED_TASKS_AND_STATES_COMPUTATION):
            comp = self._computation_class(n_tasks=len(tasks), fuse_state_tensors=fuse_states, **common, **kwargs)
            self._metrics_computations = nn.ModuleList([comp])
        else:
            self._metrics_computations = nn.ModuleList(
                [self._computation_class(n_tasks=1, fuse_state_tensors=False, **common, **kwargs) for _ in tasks]
            )

    # ---- helpers ------------------------------------------------------------------------------------
    def _fused(self) -> bool:
        return self._compute_mode in (RecComputeMode.FUSED_TASKS_COMPUTATION, RecComputeMode.FUSED_TASKS_AND_STATES_COMPUTATION)

    def _tasks_iter(self, compute_scope: str) -> Iterator[Tuple[RecTaskInfo, MetricNameBase, torch.Tensor, str, Optional[str]]]:
        """(task, metric name, value, prefix, description) of every report of every computation."""
        if self._fused():
            comp = self._metrics_computations[0]
            for rep in getattr(comp, compute_scope + "compute")():
                for task, value in zip(self._tasks, rep.value):
                    yield task, rep.name, value, compute_scope + str(rep.metric_prefix), rep.description
        else:
            for task, comp in zip(self._tasks, self._metrics_computations):
                for rep in getattr(comp, compute_scope + "compute")():
                    v = rep.value
                    yield task, rep.name, (v.squeeze(0) if v.dim() > 0 and v.shape[0] == 1 else v), compute_scope + str(rep.metric_prefix), rep.description

    def _default_weight(self, like: torch.Tensor) -> torch.Tensor:
        key = tuple(like.shape)
        w = self._default_weights.get(key)
        if w is None or w.device != like.device:
            w = torch.ones_like(like, dtype=torch.float32)
            self._default_weights[key] = w
        return w

    @staticmethod
    def _valid(weights: Optional[torch.Tensor]) -> bool:
        return weights is None or bool((weights.abs().sum(dim=-1) > 0).any())

    def _update(self, *, predictions: Optional[RecModelOutput], labels: RecModelOutput, weights: Optional[RecModelOutput], **kwargs: Any) -> None:
        with torch.no_grad():
            if self._fused():
                # tensors already stacked [n_tasks, B], or dicts to stack in task order
                def stack(x: Optional[RecModelOutput]) -> Optional[torch.Tensor]:
                    if x is None:
                        return None
                    if isinstance(x, torch.Tensor):
                        return x.view(len(self._tasks), -1) if x.dim() == 1 else x
                    return torch.stack([x[t.name].view(-1) for t in self._tasks])

                p, l, w = stack(predictions), stack(labels), stack(weights)
                assert l is not None
                if w is None:
                    w = self._default_weight(l)
                if self._should_validate_update and not self._valid(w):
                    return
                extra = {k: (torch.stack([v[t.name] for t in self._tasks]) if isinstance(v, dict) and all(t.name in v for t in self._tasks) else v) for k, v in kwargs.items()}
                self._metrics_computations[0].update(predictions=p, labels=l, weights=w, **extra)
                return
            for task, comp in zip(self._tasks, self._metrics_computations):
                if not isinstance(labels, dict) or task.name not in labels:
                    if isinstance(labels, dict):
                        continue
                l = (labels[task.name] if isinstance(labels, dict) else labels)
                p = None if predictions is None else (predictions[task.name] if isinstance(predictions, dict) else predictions)
                w = None if weights is None else (weights[task.name] if isinstance(weights, dict) else weights)
                if l.numel() == 0 and (p is None or p.numel() == 0):
                    continue
                l = l.view(1, -1) if l.dim() <= 1 else l
                if p is not None and p.dim() <= 1:
                    p = p.view(1, -1)
                if w is None:
                    w = self._default_weight(l)
                elif w.dim() <= 1:
                    w = w.view(1, -1)
                if self._should_validate_update and not self._valid(w):
                    continue
                extra = {k: (v[task.name] if isinstance(v, dict) and task.name in v else v) for k, v in kwargs.items()}
                comp.update(predictions=p, labels=l, weights=w, **extra)

    def update(self, *, predictions: Optional[RecModelOutput], labels: RecModelOutput, weights: Optional[RecModelOutput], **kwargs: Any) -> None:
        if self._fused_update_limit > 0:
            self._update_buffers[self.PREDICTIONS].append(predictions)
            self._update_buffers[self.LABELS].append(labels)
            self._update_buffers[self.WEIGHTS].append(weights)
            for k, v in kwargs.items():
                self._update_buffers.setdefault(k, []).append(v)
            if len(self._update_buffers[self.LABELS]) >= self._fused_update_limit:
                self._fused_update()
        else:
            self._update(predictions=predictions, labels=labels, weights=weights, **kwargs)

    def _fused_update(self) -> None:
        """Apply all buffered updates as one concatenated update."""
        n = len(self._update_buffers[self.LABELS])
        if n == 0:
            return

        def cat(items: List[Optional[RecModelOutput]]) -> Optional[RecModelOutput]:
            if not items or items[0] is None:
                return None
            if isinstance(items[0], dict):
                return {k: torch.cat([it[k] for it in items], dim=-1) for k in items[0].keys()}
            return torch.cat(items, dim=-1)

        merged = {k: cat(v) for k, v in self._update_buffers.items()}
        for v in self._update_buffers.values():
            v.clear()
        self._update(predictions=merged.pop(self.PREDICTIONS), labels=merged.pop(self.LABELS), weights=merged.pop(self.WEIGHTS), **merged)

    def _compose(self, compute_scope: str) -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {}
        for task, name, value, prefix, description in self._tasks_iter(compute_scope):
            # prefix string already includes lifetime_/window_; compose_metric_key concatenates verbatim
            out[f"{self._namespace}-{task.name}|{prefix}{name}{description or ''}"] = value
        return out

    def compute(self) -> Dict[str, torch.Tensor]:
        if self._fused_update_limit > 0:
            self._fused_update()
        return self._compose("")

    def local_compute(self) -> Dict[str, torch.Tensor]:
        if self._fused_update_limit > 0:
            self._fused_update()
        return self._compose("local_")

    def sync(self) -> None:
        """States are combined across ranks inside ``compute``; nothing to do ahead of it."""

    def unsync(self) -> None:
        pass

    def reset(self) -> None:
        for c in self._metrics_computations:
            c.reset()

    def get_memory_usage(self) -> Dict[torch.Tensor, int]:
        """Bytes held per state tensor (lifetime, window and queued window contributions)."""
        usage: Dict[torch.Tensor, int] = {}
        for comp in self._metrics_computations:
            for t in comp.buffers():
                usage[t] = t.numel() * t.element_size()
            for lst in comp._list_states.values():
                for t in lst:
                    usage[t] = t.numel() * t.element_size()
            if comp._batch_window_buffers:
                for wb in comp._batch_window_buffers.values():
                    for t in wb.buffers:
                        usage[t] = t.numel() * t.element_size()
        return usage

    def get_required_inputs(self) -> set:
        return self._required_inputs


class RecMetricList(nn.Module):
    """Calls ``update``/``compute`` on several ``RecMetric`` objects and merges their results."""

    rec_metrics: nn.ModuleList
    required_inputs: Optional[List[str]]

    def __init__(self, rec_metrics: List[RecMetric]) -> None:
        super().__init__()
        self.rec_metrics = nn.ModuleList(rec_metrics)
        self.required_inputs = list(set().union(*[m.get_required_inputs() for m in rec_metrics])) or None if rec_metrics else None

    def __len__(self) -> int:
        return len(self.rec_metrics)

    def __getitem__(self, idx: int) -> nn.Module:
        return self.rec_metrics[idx]

    def get_required_inputs(self) -> Optional[List[str]]:
        return self.required_inputs

    def update(self, *, predictions: Optional[RecModelOutput], labels: RecModelOutput, weights: Optional[RecModelOutput], **kwargs: Any) -> None:
        for m in self.rec_metrics:
            m.update(predictions=predictions, labels=labels, weights=weights, **kwargs)

    def compute(self) -> Dict[str, torch.Tensor]:
        ret: Dict[str, torch.Tensor] = {}
        for m in self.rec_metrics:
            ret.update(m.compute())
        return ret

    def local_compute(self) -> Dict[str, torch.Tensor]:
        ret: Dict[str, torch.Tensor] = {}
        for m in self.rec_metrics:
            ret.update(m.local_compute())
        return ret

    def sync(self) -> None:
        for m in self.rec_metrics:
            m.sync()

    def unsync(self) -> None:
        for m in self.rec_metrics:
            m.unsync()

    def reset(self) -> None:
        for m in self.rec_metrics:
            m.reset()
