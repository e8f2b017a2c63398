"""Types of the train pipelines (cf. ``torchrec/distributed/train_pipeline/types.py``)."""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum, unique
from typing import Any, Dict, List, Optional, Tuple, Union


@unique
class PipelineState(Enum):
    """Where in a step the pipeline is; used when a step must be recovered after a failure."""

    IDLE = 0
    CALL_FWD = 1
    CALL_BWD = 2

    def __str__(self) -> str:
        return self.name


@dataclass
class ArgInfo:
    """How to obtain one argument of a pipelined module: a chain of steps, each either an attribute name
    (``is_getitem=False``) or an item key (``is_getitem=True``), applied to the batch -- or, when ``postproc`` is set, to the
    output of that pipelined post-processing module for the batch.  ``constant`` (a 1-tuple) carries a literal instead."""

    input_attrs: List[Union[str, int]] = field(default_factory=list)
    is_getitems: List[bool] = field(default_factory=list)
    name: Optional[str] = None
    postproc: Optional[Any] = None
    constant: Optional[Tuple[Any]] = None

    def resolve(self, batch: Any, context: Any = None) -> Any:
        if self.constant is not None:
            return self.constant[0]
        obj = self.postproc.run(batch, context) if self.postproc is not None else batch
        for attr, is_getitem in zip(self.input_attrs, self.is_getitems):
            obj = obj[attr] if is_getitem else (getattr(obj, attr) if attr != "" else obj)
        return obj


@dataclass
class CallArgs:
    """Positional and keyword ``ArgInfo`` of one pipelined module."""

    args: List[ArgInfo] = field(default_factory=list)
    kwargs: Dict[str, ArgInfo] = field(default_factory=dict)

    def build_args_kwargs(self, batch: Any, context: Any = None) -> Tuple[List[Any], Dict[str, Any]]:
        return [a.resolve(batch, context) for a in self.args], {k: a.resolve(batch, context) for k, a in self.kwargs.items()}


@dataclass
class PipelineStageConfig:
    name: str
    stream_priority: int = 0
