"""Types of the model delta tracker (``torchrec/distributed/model_tracker/types.py:18-84``)."""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import List, Optional

import torch


@dataclass
class IndexedLookup:
    """The ids (and optionally states) one lookup touched in batch ``batch_idx``."""

    batch_idx: int
    ids: torch.Tensor
    states: Optional[torch.Tensor]


@dataclass
class DeltaRows:
    """Unique touched ids of a table and the state recorded for each."""

    ids: torch.Tensor
    states: Optional[torch.Tensor]


class TrackingMode(Enum):
    ID_ONLY = "id_only"          # which rows changed
    EMBEDDING = "embedding"      # rows + the embedding values seen by the lookup
    MOMENTUM_LAST = "momentum_last"
    MOMENTUM_DIFF = "momentum_diff"
    ROWWISE_ADAGRAD = "rowwise_adagrad"


class EmbdUpdateMode(Enum):
    NONE = "none"    # ids only
    FIRST = "first"  # keep the state of the first occurrence of an id
    LAST = "last"    # keep the state of the last occurrence


@dataclass
class ModelTrackerConfig:
    tracking_mode: TrackingMode = TrackingMode.ID_ONLY
    consumers: Optional[List[str]] = None
    delete_on_read: bool = True
    auto_compact: bool = False
    fqns_to_skip: List[str] = field(default_factory=list)
