"""``@_torchrec_method_logger()``: log the inputs of a call and its outcome (or the exception) as one structured record
(``torchrec/distributed/logger.py:24``)."""
from __future__ import annotations

import functools
import inspect
from typing import Any, Callable, Dict, TypeVar

from typing_extensions import ParamSpec

from torchrec_b200.distributed import torchrec_logger

__all__ = ["_torchrec_method_logger"]
_P = ParamSpec("_P")
_T = TypeVar("_T")


def _get_input_from_func(func: Callable, *args: Any, **kwargs: Any) -> str:
    try:
        bound = inspect.signature(func).bind_partial(*args, **kwargs)
        bound.apply_defaults()
        return str({k: (type(v).__name__ if k == "self" else repr(v)[:200]) for k, v in bound.arguments.items()})
    except Exception as e:  # the logger must never break the call it observes
        return f"<unavailable: {e}>"


def _torchrec_method_logger(**wrapper_kwargs: Any) -> Callable[[Callable[_P, _T]], Callable[_P, _T]]:
    def decorator(func: Callable[_P, _T]) -> Callable[_P, _T]:
        @functools.wraps(func)
        def wrapper(*args: _P.args, **kwargs: _P.kwargs) -> _T:
            logger = torchrec_logger._get_or_create_logger()
            msg: Dict[str, Any] = torchrec_logger._get_msg_dict(func.__name__, **kwargs)
            try:
                msg["input"] = _get_input_from_func(func, *args, **kwargs)
                result = func(*args, **kwargs)
                msg["output"] = repr(result)[:200]
                logger.debug(msg)
                return result
            except BaseException as error:
                msg["error"] = f"{error}"
                logger.error(msg)
                raise

        return wrapper

    return decorator
