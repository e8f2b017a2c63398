"""Types of the train pipelines (cf. ``torchrec/distributed/train_pipeline/types.py``)."""
from __future__ import annotations

import abc
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


class BaseArgInfoStep(abc.ABC):
    """One transformation on the way from the batch to a module argument.  An ``ArgInfo`` built from steps applies them in order,
    each to the previous one's output.  Two steps are equal when they are of one class with equal fields (so ``CallArgs`` can be
    compared in tests).  Counterpart of ``torchrec/distributed/train_pipeline/types.py:17-40`` and ``tracing.py:40-137``."""

    @abc.abstractmethod
    def process(self, arg: Any) -> Any:
        ...

    def __eq__(self, other: object) -> bool:
        return isinstance(other, type(self)) and vars(self) == vars(other)

    def __repr__(self) -> str:
        return f"{type(self).__name__}({', '.join(f'{k}={v!r}' for k, v in vars(self).items())})"


class NoopArgInfoStep(BaseArgInfoStep):
    def process(self, arg: Any) -> Any:
        return arg


class GetAttrArgInfoStep(BaseArgInfoStep):
    def __init__(self, attr_name: str) -> None:
        self.attr_name = attr_name

    def process(self, arg: Any) -> Any:
        return getattr(arg, self.attr_name)


class GetItemArgInfoStep(BaseArgInfoStep):
    def __init__(self, item_index: Union[str, int]) -> None:
        self.item_index = item_index

    def process(self, arg: Any) -> Any:
        return arg[self.item_index]


class PostprocArgInfoStep(BaseArgInfoStep):
    """Run a post-processing module on what the previous steps produced."""

    def __init__(self, postproc_module: Any) -> None:
        self.postproc_module = postproc_module

    def process(self, arg: Any) -> Any:
        return self.postproc_module(arg)


class ScalarArgInfoStep(BaseArgInfoStep):
    """A literal: the input is ignored."""

    def __init__(self, value: object) -> None:
        self.value = value

    def process(self, arg: Any) -> Any:
        return self.value


class ListArgInfoStep(BaseArgInfoStep):
    """A list argument whose elements are each described by an ``ArgInfo`` over the same input."""

    def __init__(self, value: List[object]) -> None:
        self.value = value

    def process(self, arg: Any) -> Any:
        return [v.process_steps(arg) if isinstance(v, ArgInfo) else v for v in self.value]


class DictArgInfoStep(BaseArgInfoStep):
    def __init__(self, value: Dict[str, object]) -> None:
        self.value = value

    def process(self, arg: Any) -> Any:
        return {k: (v.process_steps(arg) if isinstance(v, ArgInfo) else v) for k, v in self.value.items()}


class ArgInfoStepFactory:
    """Constructors of the steps by what they do."""

    @classmethod
    def noop(cls) -> NoopArgInfoStep:
        return NoopArgInfoStep()

    @classmethod
    def get_attr(cls, name: str) -> GetAttrArgInfoStep:
        return GetAttrArgInfoStep(name)

    @classmethod
    def get_item(cls, index: Union[str, int]) -> GetItemArgInfoStep:
        return GetItemArgInfoStep(index)

    @classmethod
    def postproc(cls, pipelined_postproc_module: Any) -> PostprocArgInfoStep:
        return PostprocArgInfoStep(pipelined_postproc_module)

    @classmethod
    def from_scalar(cls, value: object) -> ScalarArgInfoStep:
        return ScalarArgInfoStep(value)

    @classmethod
    def from_list(cls, value: List[object]) -> ListArgInfoStep:
        return ListArgInfoStep(value)

    @classmethod
    def from_dict(cls, value: Dict[str, object]) -> DictArgInfoStep:
        return DictArgInfoStep(value)


@dataclass
class ArgInfo:
    """How to obtain one argument of a pipelined module: a chain of steps, each either an attribute name
    (``is_getitem=False``) or an item key (``is_getitem=True``), applied to the batch -- or, when ``postproc`` is set, to the
    output of that pipelined post-processing module for the batch.  ``constant`` (a 1-tuple) carries a literal instead.
    Alternatively ``steps`` gives the transformations explicitly (``BaseArgInfoStep`` objects, applied in order); a hand-written
    ``CallArgs`` can use either form."""

    input_attrs: List[Union[str, int]] = field(default_factory=list)
    is_getitems: List[bool] = field(default_factory=list)
    name: Optional[str] = None
    postproc: Optional[Any] = None
    constant: Optional[Tuple[Any]] = None
    steps: Optional[List[BaseArgInfoStep]] = None

    def add_step(self, step: BaseArgInfoStep) -> "ArgInfo":
        """Put ``step`` in front of the others (it runs first)."""
        self.steps = [step] + list(self.steps or [])
        return self

    def append_step(self, step: BaseArgInfoStep) -> "ArgInfo":
        self.steps = list(self.steps or []) + [step]
        return self

    def process_steps(self, arg: Any) -> Any:
        """Apply the explicit steps to ``arg``; None when there are none."""
        if not self.steps:
            return None
        for step in self.steps:
            arg = step.process(arg)
        return arg

    def resolve(self, batch: Any, context: Any = None) -> Any:
        if self.steps is not None:
            return self.process_steps(batch)
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
