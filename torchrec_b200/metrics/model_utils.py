"""Pull labels / predictions / weights (and extra inputs) of every task out of a model-output dict
(``torchrec/metrics/model_utils.py``)."""
from __future__ import annotations

import logging
from typing import Dict, List, Optional, Tuple

import torch

from torchrec_b200.metrics.rec_metric import RecTaskInfo

logger = logging.getLogger(__name__)


def is_empty_signals(labels: torch.Tensor, predictions: torch.Tensor, weights: torch.Tensor) -> bool:
    return torch.numel(labels) <= 0 and torch.numel(predictions) <= 0 and torch.numel(weights) <= 0


def parse_model_outputs(label_name: str, prediction_name: str, weight_name: str, model_out: Dict[str, torch.Tensor]
                        ) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    labels = model_out[label_name].squeeze()
    if not prediction_name:
        assert not weight_name, "weight name must be empty if prediction name is empty"
        return labels, None, None  # type: ignore[return-value]
    assert isinstance(labels, torch.Tensor)
    predictions = model_out[prediction_name].squeeze()
    assert isinstance(predictions, torch.Tensor)
    weights = model_out[weight_name].squeeze() if weight_name else None
    if not is_empty_signals(labels, predictions, weights if weights is not None else labels):
        if labels.dim() == predictions.dim():
            assert torch.numel(labels) == torch.numel(predictions), f"Expect the same number of elements in labels and predictions. {labels.shape} vs {predictions.shape}"
        elif labels.dim() < predictions.dim():  # multiclass: predictions [B, n_classes]
            assert torch.numel(labels) == torch.numel(predictions) / predictions.size()[-1]
        else:
            assert torch.numel(labels) / labels.size()[-1] == torch.numel(predictions)
        if weights is not None:
            assert torch.numel(labels) == torch.numel(weights) or labels.dim() != predictions.dim()
    labels = labels.unsqueeze(0) if labels.dim() == 0 else labels
    predictions = predictions.unsqueeze(0) if predictions.dim() == 0 else predictions
    if weights is not None and weights.dim() == 0:
        weights = weights.unsqueeze(0)
    return labels, predictions, weights


def session_ids_to_tensor(session_ids: List[str], device: Optional[torch.device] = None) -> torch.Tensor:
    """Session names of consecutive examples to run numbers: 1 for the first run of equal names, 2 for the next, ...
    (``["a", "a", "b", "a"]`` -> ``[1, 1, 2, 3]``); the form the session metrics take their grouping in
    (``torchrec/metrics/model_utils.py:20-38``)."""
    runs: List[int] = []
    current = 0
    previous: object = object()
    for name in session_ids:
        if name != previous:
            current += 1
            previous = name
        runs.append(current)
    return torch.tensor(runs, device=device)


def parse_required_inputs(model_out: Dict[str, torch.Tensor], required_inputs_list: List[str], ndcg_transform_input: bool = False,
                          device: Optional[torch.device] = None) -> Dict[str, torch.Tensor]:
    required_inputs: Dict[str, torch.Tensor] = {}
    for feature in required_inputs_list:
        if feature not in model_out:
            continue
        value = model_out[feature]
        if ndcg_transform_input and isinstance(value, list):
            value = model_out[feature] = session_ids_to_tensor(value, device=device)
        t = value.squeeze()
        assert isinstance(t, torch.Tensor)
        required_inputs[feature] = t.to(device) if device is not None else t
    return required_inputs


def parse_task_model_outputs(tasks: List[RecTaskInfo], model_out: Dict[str, torch.Tensor], required_inputs_list: Optional[List[str]] = None
                             ) -> Tuple[Dict[str, torch.Tensor], Dict[str, torch.Tensor], Dict[str, torch.Tensor], Dict[str, torch.Tensor]]:
    all_labels: Dict[str, torch.Tensor] = {}
    all_predictions: Dict[str, torch.Tensor] = {}
    all_weights: Dict[str, torch.Tensor] = {}
    all_required_inputs: Dict[str, torch.Tensor] = {}
    for task in tasks:
        labels, predictions, weights = parse_model_outputs(task.label_name, task.prediction_name, task.weight_name, model_out)
        if predictions is not None and predictions.numel() > 0:  # skip tasks without data this batch
            all_predictions[task.name] = predictions
        if labels.numel() > 0 or predictions is None:
            all_labels[task.name] = labels
        if weights is not None and weights.numel() > 0:
            all_weights[task.name] = weights
    if required_inputs_list:
        all_required_inputs = parse_required_inputs(model_out, required_inputs_list)
    return all_labels, all_predictions, all_weights, all_required_inputs
