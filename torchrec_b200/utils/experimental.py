"""``@experimental`` marks an API as unstable: the first call logs one warning (``torchrec/utils/experimental.py``)."""
from __future__ import annotations

import functools
import inspect
import warnings
from typing import Any, Callable, Optional, TypeVar, Union

F = TypeVar("F", bound=Callable[..., Any])


def experimental(obj: Optional[Union[F, type]] = None, *, feature: Optional[str] = None, since: Optional[str] = None) -> Any:
    def decorate(target: Any) -> Any:
        name = feature or getattr(target, "__qualname__", str(target))
        msg = f"`{name}` is *experimental*" + (f" (since {since})" if since else "") + " and may change or be removed without notice."
        warned = {"done": False}

        def warn() -> None:
            if not warned["done"]:
                warned["done"] = True
                warnings.warn(msg, UserWarning, stacklevel=3)

        if inspect.isclass(target):
            orig = target.__init__

            @functools.wraps(orig)
            def init(self, *a: Any, **k: Any) -> None:
                warn()
                orig(self, *a, **k)

            target.__init__ = init
            return target

        @functools.wraps(target)
        def wrapper(*a: Any, **k: Any) -> Any:
            warn()
            return target(*a, **k)

        return wrapper

    return decorate(obj) if obj is not None else decorate
