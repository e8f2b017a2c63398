"""Event hooks of in-training embedding pruning: a context manager per event whose attributes a deployment can ship to its own
telemetry.  The default records nothing.  Counterpart of ``torchrec/modules/pruning_logger.py``."""
from __future__ import annotations

from abc import ABC, abstractmethod
from contextlib import contextmanager
from typing import Any, Iterator, Optional


class PruningLogBase(object):
    """Marker base for what a logger yields."""


class PruningLogDetails(PruningLogBase):
    """Attribute bag filled inside ``with pruning_logger(...) as details``."""

    def __setattr__(self, name: str, value: Any) -> None:
        object.__setattr__(self, name, value)


class PruningLogger(ABC):
    @classmethod
    @abstractmethod
    def pruning_logger(cls, event: str, trainer: Optional[str] = None, publisher: Optional[str] = None) -> Any:
        ...


class PruningLoggerDefault(PruningLogger):
    @classmethod
    @contextmanager
    def pruning_logger(cls, event: str, trainer: Optional[str] = None, publisher: Optional[str] = None) -> Iterator[PruningLogDetails]:
        yield PruningLogDetails()
