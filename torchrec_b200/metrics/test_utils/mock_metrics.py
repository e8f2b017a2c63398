"""Helpers for tests of the metric module's state handling: dictionaries of tensor states and a deep comparison
(``torchrec/metrics/test_utils/mock_metrics.py:226-310``)."""
from __future__ import annotations

from typing import Any, Dict, List

import torch


def create_tensor_states(keys: List[str], n_tasks: int = 1) -> Dict[str, Any]:
    return {k: torch.rand(n_tasks, dtype=torch.double) for k in keys}


def create_tensor_list_states(keys: List[str]) -> Dict[str, Any]:
    return {k: [torch.rand(1, 4, dtype=torch.double), torch.rand(1, 3, dtype=torch.double)] for k in keys}


def create_metric_states_dict(metric_prefix: str, computation_name: str, metric_states: Dict[str, Any]) -> Dict[str, Any]:
    """State-dict style keys of one computation of one metric."""
    return {f"{metric_prefix}.{computation_name}.{k}": v for k, v in metric_states.items()}


def assert_tensor_dict_equals(actual: Dict[str, Any], expected: Dict[str, Any], path: str = "") -> None:
    assert actual.keys() == expected.keys(), f"{path}: {sorted(actual)} != {sorted(expected)}"
    for k, e in expected.items():
        a = actual[k]
        where = f"{path}.{k}" if path else k
        if isinstance(e, dict):
            assert_tensor_dict_equals(a, e, where)
        elif isinstance(e, (list, tuple)):
            assert len(a) == len(e), where
            for i, (x, y) in enumerate(zip(a, e)):
                torch.testing.assert_close(x, y, msg=lambda m: f"{where}[{i}]: {m}")
        elif isinstance(e, torch.Tensor):
            torch.testing.assert_close(a, e, msg=lambda m: f"{where}: {m}")
        else:
            assert a == e, where
