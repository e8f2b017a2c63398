"""Naming of reported metrics: ``"<namespace>-<task>|<prefix><metric name><description>"``.

Namespace = which metric object produced the value, task = user task name, prefix = lifetime / window /
attempt.  Same key format and vocabulary as ``torchrec/metrics/metrics_namespace.py`` so dashboards and
checkpoints written against either framework line up.
"""
from __future__ import annotations

from enum import Enum
from typing import Optional


class StrValueMixin:
    def __str__(self) -> str:
        return self.value  # type: ignore[attr-defined]


class MetricNameBase(StrValueMixin, Enum):
    pass


def _names(cls_name: str, base, values: str):
    """Enum from a whitespace-separated ``NAME=value`` table (``NAME`` alone means value = name.lower())."""
    members = {}
    for tok in values.split():
        k, _, v = tok.partition("=")
        members[k] = v if _ else k.lower()
    return base(cls_name, members)


MetricName = _names(
    "MetricName", MetricNameBase,
    "DEFAULT= NE NE_POSITIVE SEGMENTED_NE LOG_LOSS=logloss THROUGHPUT TOTAL_EXAMPLES ATTEMPT_EXAMPLES BATCH_SIZE CTR CALIBRATION "
    "MSE MAE RMSE R_SQUARED AUC GAUC AUPRC RAUC GROUPED_AUC GROUPED_AUPRC GROUPED_RAUC RECALL_SESSION_LEVEL "
    "PRECISION_SESSION_LEVEL MULTICLASS_RECALL WEIGHTED_AVG TOWER_QPS=qps ACCURACY NDCG XAUC SCALAR OUTPUT GAUC_NUM_SAMPLES "
    "TOTAL_POSITIVE_EXAMPLES TOTAL_NEGATIVE_EXAMPLES PRECISION RECALL SERVING_NE SERVING_CALIBRATION TENSOR_WEIGHTED_AVG "
    "CALI_FREE_NE UNWEIGHTED_NE HINDSIGHT_TARGET_PR HINDSIGHT_TARGET_PRECISION HINDSIGHT_TARGET_RECALL EFFECTIVE_SAMPLE_RATE "
    "RECALIBRATED_NE RECALIBRATED_CALIBRATION",
)


class MetricNamespaceBase(StrValueMixin, Enum):
    pass


MetricNamespace = _names(
    "MetricNamespace", MetricNamespaceBase,
    "DEFAULT= NE NE_POSITIVE SEGMENTED_NE RECALIBRATED_NE RECALIBRATED_CALIBRATION THROUGHPUT CTR CALIBRATION MSE AUC GAUC AUPRC "
    "RAUC MAE ACCURACY OPTIMIZERS MODEL_CONFIGURATOR MULTICLASS_RECALL WEIGHTED_AVG RECALL_SESSION_LEVEL PRECISION_SESSION_LEVEL "
    "TOWER_QPS=qps NDCG XAUC SCALAR PRECISION RECALL SERVING_NE SERVING_CALIBRATION OUTPUT TENSOR_WEIGHTED_AVG CALI_FREE_NE "
    "UNWEIGHTED_NE HINDSIGHT_TARGET_PR EFFECTIVE_RATE",
)


class MetricPrefix(StrValueMixin, Enum):
    DEFAULT = ""
    LIFETIME = "lifetime_"
    WINDOW = "window_"
    ATTEMPT = "attempt_"


def task_wildcard_metrics_pattern(namespace, metric_name, metric_prefix: MetricPrefix = MetricPrefix.DEFAULT) -> str:
    """Regex matching one metric of a namespace for any task."""
    return rf"{namespace}-.+\|{metric_prefix}{metric_name}"


def compose_metric_namespace(namespace, task_name: str) -> str:
    return f"{namespace}-{task_name}"


def compose_customized_metric_key(namespace: str, metric_name: str, description: Optional[str] = None) -> str:
    return f"{namespace}|{metric_name}{description or ''}"


def compose_metric_key(namespace, task_name: str, metric_name, metric_prefix: MetricPrefix = MetricPrefix.DEFAULT,
                       description: Optional[str] = None) -> str:
    return compose_customized_metric_key(compose_metric_namespace(namespace, task_name), f"{metric_prefix}{metric_name}", description)
