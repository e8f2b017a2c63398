"""Harness for metric tests: synthetic batches and tasks, a reference-metric base class, and helpers that run a metric next to
its reference over a stream of batches and compare lifetime and window values.

A reference metric (``TestMetric`` subclass) states what the metric means in two static methods: ``_get_states`` turns one batch
into a dictionary of additive tensors and ``_compute`` turns accumulated states into the value.  The harness keeps lifetime sums and
the sums of the batches inside the window, so any metric whose states add up can be checked against a few lines of plain torch.
Counterpart of ``torchrec/metrics/test_utils/__init__.py:35-700``."""
from __future__ import annotations

import abc
import random
from typing import Any, Dict, List, Optional, Tuple, Type, Union

import torch

from torchrec_b200.metrics.metrics_config import RecComputeMode, RecTaskInfo
from torchrec_b200.metrics.rec_metric import RecMetric


def gen_test_batch(batch_size: int, label_name: str = "label", prediction_name: str = "prediction", weight_name: str = "weight", tensor_name: str = "tensor",
                   mask_tensor_name: Optional[str] = None, label_value: Optional[torch.Tensor] = None, prediction_value: Optional[torch.Tensor] = None,
                   weight_value: Optional[torch.Tensor] = None, mask: Optional[torch.Tensor] = None, n_classes: Optional[int] = None,
                   seed: Optional[int] = None, device: Optional[Union[str, torch.device]] = None) -> Dict[str, torch.Tensor]:
    """One batch as ``{name: float64 tensor}``; values are random unless given."""
    device = torch.device(device or "cpu")
    gen = torch.Generator()
    gen.manual_seed(seed if seed is not None else random.getrandbits(31))
    label = label_value if label_value is not None else torch.randint(0, n_classes or 2, (batch_size,), generator=gen).double()
    shape = (batch_size,) if n_classes is None else (batch_size, n_classes)
    prediction = prediction_value if prediction_value is not None else torch.rand(shape, dtype=torch.double, generator=gen)
    weight = weight_value if weight_value is not None else torch.rand(batch_size, dtype=torch.double, generator=gen)
    batch = {label_name: label.to(device), prediction_name: prediction.to(device), weight_name: weight.to(device),
             tensor_name: torch.rand(batch_size, dtype=torch.double, generator=gen).to(device)}
    if mask_tensor_name is not None:
        batch[mask_tensor_name] = (mask if mask is not None else torch.ones(batch_size, dtype=torch.double)).to(device)
    return batch


def gen_test_tasks(task_names: List[str]) -> List[RecTaskInfo]:
    return [RecTaskInfo(name=n, label_name=f"{n}-label", prediction_name=f"{n}-prediction", weight_name=f"{n}-weight", tensor_name=f"{n}-tensor") for n in task_names]


def gen_test_timestamps(nsteps: int) -> List[float]:
    out, t = [], 0.0
    for _ in range(nsteps):
        out.append(t)
        t += random.uniform(1.0, 5.0)
    return out


class TestMetric(abc.ABC):
    """Reference metric: additive states per task, lifetime and windowed."""

    __test__ = False

    def __init__(self, world_size: int, rec_tasks: List[RecTaskInfo], compute_lifetime_metric: bool = True, compute_window_metric: bool = True,
                 local_compute_lifetime_metric: bool = True, local_compute_window_metric: bool = True) -> None:
        self.world_size = world_size
        self._rec_tasks = rec_tasks
        self._compute_lifetime_metric, self._compute_window_metric = compute_lifetime_metric, compute_window_metric

    @staticmethod
    @abc.abstractmethod
    def _get_states(labels: torch.Tensor, predictions: torch.Tensor, weights: torch.Tensor, required_inputs_tensor: Optional[torch.Tensor] = None) -> Dict[str, torch.Tensor]: ...

    @staticmethod
    @abc.abstractmethod
    def _compute(states: Dict[str, torch.Tensor]) -> torch.Tensor: ...

    @staticmethod
    def _sum(states: List[Dict[str, torch.Tensor]]) -> Dict[str, torch.Tensor]:
        return {k: sum(s[k] for s in states) for k in states[0]}

    def compute(self, model_outs: List[Dict[str, torch.Tensor]], nsteps: int, batch_window_size: int, timestamps: Optional[List[float]] = None) -> Tuple[Dict[str, torch.Tensor], Dict[str, torch.Tensor]]:
        """``(lifetime value per task, window value per task)`` after ``nsteps`` batches; the window covers the last
        ``batch_window_size`` batches."""
        lifetime, window = {}, {}
        for task in self._rec_tasks:
            per_step = []
            for i in range(nsteps):
                out = model_outs[i]
                per_step.append(self._get_states(out[task.label_name], out[task.prediction_name], out[task.weight_name],
                                                 out.get(task.tensor_name) if task.tensor_name else None))
            if self._compute_lifetime_metric:
                lifetime[task.name] = self._compute(self._sum(per_step))
            if self._compute_window_metric:
                window[task.name] = self._compute(self._sum(per_step[-batch_window_size:]))
        return lifetime, window


def rec_metric_value_test_helper(target_clazz: Type[RecMetric], target_compute_mode: RecComputeMode, test_clazz: Optional[Type[TestMetric]], fused_update_limit: int,
                                 compute_on_all_ranks: bool, should_validate_update: bool, world_size: int, my_rank: int, task_names: List[str],
                                 batch_size: int = 32, nsteps: int = 6, batch_window_size: int = 3, is_time_dependent: bool = False, time_dependent_metric=None,
                                 n_classes: Optional[int] = None, **kwargs: Any) -> Tuple[Dict[str, torch.Tensor], Tuple[Dict[str, torch.Tensor], ...]]:
    """Feed ``nsteps`` random batches to ``target_clazz`` and to the reference; returns ``(target.compute(), reference results)``."""
    tasks = gen_test_tasks(task_names)
    model_outs = []
    for step in range(nsteps):
        merged: Dict[str, torch.Tensor] = {}
        for t, task in enumerate(tasks):
            merged.update(gen_test_batch(batch_size, task.label_name, task.prediction_name, task.weight_name, task.tensor_name or "tensor",
                                         n_classes=n_classes, seed=1000 * my_rank + 10 * step + t))
        model_outs.append(merged)
    target = target_clazz(world_size=world_size, my_rank=my_rank, batch_size=batch_size, tasks=tasks, compute_mode=target_compute_mode,
                          window_size=batch_window_size * world_size * batch_size, fused_update_limit=fused_update_limit,
                          compute_on_all_ranks=compute_on_all_ranks, should_validate_update=should_validate_update, **kwargs)
    for out in model_outs:
        extra = {"required_inputs": {t.tensor_name: out[t.tensor_name] for t in tasks if t.tensor_name}} if getattr(target, "_required_inputs", None) else {}
        target.update(predictions={t.name: out[t.prediction_name] for t in tasks}, labels={t.name: out[t.label_name] for t in tasks},
                      weights={t.name: out[t.weight_name] for t in tasks}, **extra)
    result = target.compute()
    reference: Tuple[Dict[str, torch.Tensor], ...] = ()
    if test_clazz is not None:
        reference = test_clazz(world_size, tasks).compute(model_outs, nsteps, batch_window_size)
    return result, reference


def _assert_metric_results(target: Dict[str, torch.Tensor], reference: Tuple[Dict[str, torch.Tensor], ...], namespace: str, metric_name: str, task_names: List[str]) -> None:
    lifetime, window = reference
    for task in task_names:
        for prefix, ref in (("lifetime_", lifetime), ("window_", window)):
            key = f"{namespace}-{task}|{prefix}{metric_name}"
            assert key in target, (key, sorted(target))
            torch.testing.assert_close(target[key].double().reshape(-1)[0], ref[task].double().reshape(-1)[0], rtol=1e-6, atol=1e-8, msg=lambda m: f"{key}: {m}")


def rec_metric_value_test_launcher(target_clazz: Type[RecMetric], target_compute_mode: RecComputeMode, test_clazz: Type[TestMetric], metric_name: str,
                                   task_names: List[str], fused_update_limit: int = 0, compute_on_all_ranks: bool = False, should_validate_update: bool = False,
                                   world_size: int = 1, batch_size: int = 32, nsteps: int = 6, batch_window_size: int = 3, **kwargs: Any) -> None:
    """Single-process check of one metric class in one compute mode against its reference (``world_size`` must be 1 here; cross-rank
    agreement is tested by running ``rec_metric_value_test_helper`` on every rank of a spawned group)."""
    assert world_size == 1, "spawn ranks and call rec_metric_value_test_helper on each for world_size > 1"
    result, reference = rec_metric_value_test_helper(target_clazz, target_compute_mode, test_clazz, fused_update_limit, compute_on_all_ranks, should_validate_update,
                                                     1, 0, task_names, batch_size, nsteps, batch_window_size, **kwargs)
    namespace = str(target_clazz._namespace.value if hasattr(target_clazz._namespace, "value") else target_clazz._namespace)
    _assert_metric_results(result, reference, namespace, metric_name, task_names)
