"""``RecMetricModule``: all metrics of a training job behind ``update(model_out)`` / ``compute()``.

Owns the ``RecMetricList``, the ``ThroughputMetric`` and optional state metrics (optimizer / configurator
introspection); knows when to compute (every ``compute_interval_steps`` batches, with the interval re-tuned from
the measured compute time to stay between ``min/max_compute_interval`` seconds, agreed on across ranks).
``generate_metric_module`` builds one from a ``MetricsConfig``.  Counterpart of ``torchrec/metrics/metric_module.py``.
"""
from __future__ import annotations

import abc
import logging
import time
from typing import Any, Dict, List, Optional, Type, Union

import torch
import torch.distributed as dist
from torch import nn

from torchrec_b200.metrics.accuracy import AccuracyMetric
from torchrec_b200.metrics.auc import AUCMetric
from torchrec_b200.metrics.auprc import AUPRCMetric
from torchrec_b200.metrics.cali_free_ne import CaliFreeNEMetric
from torchrec_b200.metrics.calibration import CalibrationMetric
from torchrec_b200.metrics.calibration_with_recalibration import RecalibratedCalibrationMetric
from torchrec_b200.metrics.ctr import CTRMetric
from torchrec_b200.metrics.gauc import GAUCMetric
from torchrec_b200.metrics.hindsight_target_pr import HindsightTargetPRMetric
from torchrec_b200.metrics.mae import MAEMetric
from torchrec_b200.metrics.metrics_config import (
    BatchSizeStage, MetricsConfig, RecMetricEnum, RecMetricEnumBase, RecTaskInfo, StateMetricEnum, validate_batch_size_stages,
)
from torchrec_b200.metrics.metrics_namespace import compose_customized_metric_key
from torchrec_b200.metrics.model_utils import parse_task_model_outputs
from torchrec_b200.metrics.mse import MSEMetric
from torchrec_b200.metrics.multiclass_recall import MulticlassRecallMetric
from torchrec_b200.metrics.ndcg import NDCGMetric
from torchrec_b200.metrics.ne import NEMetric
from torchrec_b200.metrics.ne_positive import NEPositiveMetric
from torchrec_b200.metrics.ne_with_recalibration import RecalibratedNEMetric
from torchrec_b200.metrics.output import OutputMetric
from torchrec_b200.metrics.precision import PrecisionMetric
from torchrec_b200.metrics.precision_session import PrecisionSessionMetric
from torchrec_b200.metrics.rauc import RAUCMetric
from torchrec_b200.metrics.rec_metric import RecMetric, RecMetricList
from torchrec_b200.metrics.recall import RecallMetric
from torchrec_b200.metrics.recall_session import RecallSessionMetric
from torchrec_b200.metrics.scalar import ScalarMetric
from torchrec_b200.metrics.segmented_ne import SegmentedNEMetric
from torchrec_b200.metrics.serving_calibration import ServingCalibrationMetric
from torchrec_b200.metrics.serving_ne import ServingNEMetric
from torchrec_b200.metrics.tensor_weighted_avg import TensorWeightedAvgMetric
from torchrec_b200.metrics.throughput import ThroughputMetric
from torchrec_b200.metrics.tower_qps import TowerQPSMetric
from torchrec_b200.metrics.unweighted_ne import UnweightedNEMetric
from torchrec_b200.metrics.weighted_avg import WeightedAvgMetric
from torchrec_b200.metrics.xauc import XAUCMetric

logger = logging.getLogger(__name__)

REC_METRICS_MAPPING: Dict[RecMetricEnumBase, Type[RecMetric]] = {
    RecMetricEnum.NE: NEMetric, RecMetricEnum.NE_POSITIVE: NEPositiveMetric, RecMetricEnum.SEGMENTED_NE: SegmentedNEMetric,
    RecMetricEnum.RECALIBRATED_NE: RecalibratedNEMetric, RecMetricEnum.RECALIBRATED_CALIBRATION: RecalibratedCalibrationMetric,
    RecMetricEnum.LOG_LOSS: NEMetric, RecMetricEnum.CTR: CTRMetric, RecMetricEnum.CALIBRATION: CalibrationMetric, RecMetricEnum.AUC: AUCMetric,
    RecMetricEnum.AUPRC: AUPRCMetric, RecMetricEnum.RAUC: RAUCMetric, RecMetricEnum.GAUC: GAUCMetric, RecMetricEnum.MSE: MSEMetric,
    RecMetricEnum.MAE: MAEMetric, RecMetricEnum.MULTICLASS_RECALL: MulticlassRecallMetric, RecMetricEnum.WEIGHTED_AVG: WeightedAvgMetric,
    RecMetricEnum.TOWER_QPS: TowerQPSMetric, RecMetricEnum.RECALL_SESSION_LEVEL: RecallSessionMetric,
    RecMetricEnum.PRECISION_SESSION_LEVEL: PrecisionSessionMetric, RecMetricEnum.ACCURACY: AccuracyMetric, RecMetricEnum.NDCG: NDCGMetric,
    RecMetricEnum.XAUC: XAUCMetric, RecMetricEnum.SCALAR: ScalarMetric, RecMetricEnum.PRECISION: PrecisionMetric, RecMetricEnum.RECALL: RecallMetric,
    RecMetricEnum.SERVING_NE: ServingNEMetric, RecMetricEnum.SERVING_CALIBRATION: ServingCalibrationMetric, RecMetricEnum.OUTPUT: OutputMetric,
    RecMetricEnum.TENSOR_WEIGHTED_AVG: TensorWeightedAvgMetric, RecMetricEnum.CALI_FREE_NE: CaliFreeNEMetric,
    RecMetricEnum.UNWEIGHTED_NE: UnweightedNEMetric, RecMetricEnum.HINDSIGHT_TARGET_PR: HindsightTargetPRMetric,
}

MODEL_METRIC_LABEL: str = "model"
MEMORY_AVG_WARNING_PERCENTAGE = 20
MEMORY_AVG_WARNING_WARMUP = 100
MetricValue = Union[torch.Tensor, float]


class StateMetric(abc.ABC):
    """Values read from a training object (optimizer, configurator) at compute time, reported with the metrics."""

    @abc.abstractmethod
    def get_metrics(self) -> Dict[str, MetricValue]:
        ...


class RecMetricModule(nn.Module):
    batch_size: int
    world_size: int
    rec_tasks: List[RecTaskInfo]
    rec_metrics: RecMetricList
    throughput_metric: Optional[ThroughputMetric]
    state_metrics: Dict[str, StateMetric]

    def __init__(self, batch_size: int, world_size: int, rec_tasks: Optional[List[RecTaskInfo]] = None, rec_metrics: Optional[RecMetricList] = None,
                 throughput_metric: Optional[ThroughputMetric] = None, state_metrics: Optional[Dict[str, StateMetric]] = None,
                 compute_interval_steps: int = 100, min_compute_interval: float = 0.0, max_compute_interval: float = float("inf")) -> None:
        super().__init__()
        self.batch_size, self.world_size = batch_size, world_size
        self.rec_tasks = list(rec_tasks or [])
        self.rec_metrics = rec_metrics or RecMetricList([])
        self.throughput_metric = throughput_metric
        self.state_metrics = dict(state_metrics or {})
        self.trained_batches = self.oom_count = self.compute_count = 0
        self.compute_interval_steps = compute_interval_steps
        self.last_compute_time = -1.0
        # time bounds on the compute interval are either both left at their defaults (switched off, stored as -1) or validated
        timed = (min_compute_interval, max_compute_interval) != (0.0, float("inf"))
        if timed and max_compute_interval <= 0.0:
            raise ValueError("Max compute interval should not be smaller than or equal to 0.")
        if timed and min_compute_interval < 0.0:
            raise ValueError("Min compute interval should not be smaller than 0.")
        self.min_compute_interval, self.max_compute_interval = (min_compute_interval, max_compute_interval) if timed else (-1.0, -1.0)

    def _update_rec_metrics(self, model_out: Dict[str, torch.Tensor], **kwargs: Any) -> None:
        if not (self.rec_metrics and self.rec_tasks):
            return
        labels, predictions, weights, extra = parse_task_model_outputs(self.rec_tasks, model_out, self.get_required_inputs())
        if extra:
            kwargs["required_inputs"] = extra
        self.rec_metrics.update(predictions=predictions, labels=labels, weights=weights, **kwargs)

    def update(self, model_out: Dict[str, torch.Tensor], **kwargs: Any) -> None:
        """Feed one batch of model outputs to every metric and count it for throughput."""
        self._update_rec_metrics(model_out, **kwargs)
        self.trained_batches += 1
        if self.throughput_metric is not None:
            self.throughput_metric.update()

    def _adjust_compute_interval(self) -> None:
        """After the second compute: steps-per-interval from the measured time per step, the same on every rank."""
        if self.last_compute_time > 0 and self.min_compute_interval >= 0:
            now = time.time()
            per_step = (now - self.last_compute_time) / max(self.compute_interval_steps, 1)
            step_tensor = torch.tensor([per_step], dtype=torch.double)
            if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
                dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")
                step_tensor = step_tensor.to(dev)
                dist.all_reduce(step_tensor, op=dist.ReduceOp.MAX)
            per_step = float(step_tensor.item())
            if per_step > 0:
                lo = self.min_compute_interval / per_step
                hi = self.max_compute_interval / per_step if self.max_compute_interval != float("inf") else float("inf")
                steps = self.compute_interval_steps
                if steps < lo:
                    steps = int(lo) + 1
                if steps > hi:
                    steps = max(int(hi), 1)
                self.compute_interval_steps = max(int(steps), 1)
        self.last_compute_time = time.time()

    def should_compute(self) -> bool:
        return self.trained_batches % self.compute_interval_steps == 0

    def _throughput_values(self) -> Dict[str, MetricValue]:
        return dict(self.throughput_metric.compute()) if self.throughput_metric is not None else {}

    def compute(self) -> Dict[str, MetricValue]:
        """All metric values; every rank must call it (the states are combined across ranks)."""
        self.compute_count += 1
        values: Dict[str, MetricValue] = {}
        if self.rec_metrics:
            self._adjust_compute_interval()
            values.update(self.rec_metrics.compute())
        values.update(self._throughput_values())
        for namespace, component in self.state_metrics.items():
            for key, value in component.get_metrics().items():
                values[compose_customized_metric_key(namespace, key)] = value
        return values

    def local_compute(self) -> Dict[str, MetricValue]:
        values: Dict[str, MetricValue] = dict(self.rec_metrics.local_compute()) if self.rec_metrics else {}
        values.update(self._throughput_values())
        return values

    def sync(self) -> None:
        self.rec_metrics.sync()

    def unsync(self) -> None:
        self.rec_metrics.unsync()

    def reset(self) -> None:
        self.rec_metrics.reset()

    def get_required_inputs(self) -> Optional[List[str]]:
        return self.rec_metrics.get_required_inputs()

    def get_memory_usage(self) -> int:
        """Bytes held by all metric states (tensors counted once)."""
        total, seen = 0, set()
        for m in self.rec_metrics.rec_metrics:
            for t, n in m.get_memory_usage().items():
                if id(t) not in seen:
                    seen.add(id(t))
                    total += n
        return total

    def check_memory_usage(self, compute_count: int) -> None:
        usage = self.get_memory_usage()
        if torch.cuda.is_available():
            total = torch.cuda.get_device_properties(0).total_memory
            if compute_count > MEMORY_AVG_WARNING_WARMUP and usage > total * MEMORY_AVG_WARNING_PERCENTAGE / 100:
                logger.warning(f"RecMetricModule states use {usage / 2**30:.2f} GiB")

    # ---- snapshot of the reduced states (for checkpoints written by one rank) -------------------------
    def get_pre_compute_states(self, pg: Optional[dist.ProcessGroup] = None) -> Dict[str, Dict[str, Dict[str, Any]]]:
        """``{metric: {task: {state: tensor}}}`` of the local states (lists concatenated)."""
        out: Dict[str, Dict[str, Dict[str, Any]]] = {}
        for metric in self.rec_metrics.rec_metrics:
            per_task: Dict[str, Dict[str, Any]] = {}
            comps = metric._metrics_computations
            names = [t.name for t in metric._tasks] if len(comps) == len(metric._tasks) else ["__fused__"]
            for name, comp in zip(names, comps):
                st: Dict[str, Any] = {}
                for s in comp._state_names:
                    st[s] = [t.clone() for t in comp._list_states[s]] if s in comp._list_states else getattr(comp, s).clone()
                per_task[name] = st
            out[str(metric._namespace)] = per_task
        return out

    def load_pre_compute_states(self, source: Dict[str, Dict[str, Dict[str, Any]]]) -> None:
        for metric in self.rec_metrics.rec_metrics:
            per_task = source.get(str(metric._namespace))
            if per_task is None:
                continue
            comps = metric._metrics_computations
            names = [t.name for t in metric._tasks] if len(comps) == len(metric._tasks) else ["__fused__"]
            for name, comp in zip(names, comps):
                for s, v in per_task.get(name, {}).items():
                    if s in comp._list_states:
                        comp._list_states[s] = [t.clone() for t in v]
                    else:
                        getattr(comp, s).copy_(v)


def _generate_rec_metrics(metrics_config: MetricsConfig, world_size: int, my_rank: int, batch_size: int,
                          process_group: Optional[dist.ProcessGroup] = None, batch_size_stages: Optional[List[BatchSizeStage]] = None) -> RecMetricList:
    shared = dict(world_size=world_size, my_rank=my_rank, batch_size=batch_size, compute_mode=metrics_config.rec_compute_mode,
                  fused_update_limit=metrics_config.fused_update_limit, compute_on_all_ranks=metrics_config.compute_on_all_ranks,
                  should_validate_update=metrics_config.should_validate_update, process_group=process_group)

    def tasks_of(metric_def) -> List[RecTaskInfo]:
        by_object, by_index = metric_def.rec_tasks, metric_def.rec_task_indices
        if by_object and by_index:
            raise ValueError("Only one of RecMetricDef.rec_tasks and RecMetricDef.rec_task_indices should be specified.")
        if not by_object and not by_index:
            raise ValueError("One of RecMetricDef.rec_tasks and RecMetricDef.rec_task_indices should be a non-empty list")
        return by_object or [metrics_config.rec_tasks[i] for i in by_index]

    built = []
    for kind, metric_def in metrics_config.rec_metrics.items():
        own = dict(metric_def.arguments or {}) if metric_def else {}
        if kind == RecMetricEnum.LOG_LOSS:  # log loss is the NE computation with one more output
            own["include_logloss"] = True
        built.append(REC_METRICS_MAPPING[kind](tasks=tasks_of(metric_def), window_size=metric_def.window_size, **shared, **own))
    return RecMetricList(built)


STATE_METRICS_NAMESPACE_MAPPING: Dict[StateMetricEnum, str] = {
    StateMetricEnum.OPTIMIZERS: "optimizers", StateMetricEnum.MODEL_CONFIGURATOR: "model_configurator",
}


def _generate_state_metrics(metrics_config: MetricsConfig, state_metrics_mapping: Dict[StateMetricEnum, StateMetric]) -> Dict[str, StateMetric]:
    out: Dict[str, StateMetric] = {}
    for metric_enum in metrics_config.state_metrics:
        out[STATE_METRICS_NAMESPACE_MAPPING[metric_enum]] = state_metrics_mapping[metric_enum]
    return out


def generate_metric_module(metric_class: Type[RecMetricModule], metrics_config: MetricsConfig, batch_size: int, world_size: int, my_rank: int,
                           state_metrics_mapping: Dict[StateMetricEnum, StateMetric], device: torch.device,
                           process_group: Optional[dist.ProcessGroup] = None, batch_size_stages: Optional[List[BatchSizeStage]] = None) -> RecMetricModule:
    """Build the metric module described by ``metrics_config`` and move it to ``device``."""
    validate_batch_size_stages(batch_size_stages)
    cfg = metrics_config
    throughput = None
    if cfg.throughput_metric:
        throughput = ThroughputMetric(batch_size=batch_size, world_size=world_size, window_seconds=cfg.throughput_metric.window_size,
                                      warmup_steps=cfg.throughput_metric.warmup_steps, batch_size_stages=batch_size_stages)
    module = metric_class(
        batch_size=batch_size, world_size=world_size, rec_tasks=cfg.rec_tasks,
        rec_metrics=_generate_rec_metrics(cfg, world_size, my_rank, batch_size, process_group, batch_size_stages), throughput_metric=throughput,
        state_metrics=_generate_state_metrics(cfg, state_metrics_mapping), compute_interval_steps=cfg.compute_interval_steps,
        min_compute_interval=cfg.min_compute_interval, max_compute_interval=cfg.max_compute_interval,
    )
    return module.to(device)
