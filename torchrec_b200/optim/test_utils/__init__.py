"""Optimizer fixtures for tests (``torchrec/optim/test_utils/__init__.py:15``)."""
from typing import Any

from torchrec_b200.optim.keyed import KeyedOptimizer


class DummyKeyedOptimizer(KeyedOptimizer):
    """A keyed optimizer whose ``step`` does nothing: tests drive ``state`` / ``param_groups`` by hand."""

    def __init__(self, *args: Any, **kwargs: Any) -> None:
        super().__init__(*args, **kwargs)

    def step(self, closure: Any = None) -> None:
        return None
