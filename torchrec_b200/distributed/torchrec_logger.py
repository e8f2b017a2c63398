"""Structured logger for API-usage events (``torchrec/distributed/torchrec_logger.py``)."""
from __future__ import annotations

import logging
from typing import Any, Dict

import torch.distributed as dist

from torchrec_b200.distributed.logging_handlers import _log_handlers

_DEFAULT_DESTINATION = "default"


def _get_logging_handler(destination: str = _DEFAULT_DESTINATION) -> tuple:
    handler = _log_handlers[destination]
    return handler, f"{type(handler).__name__}-{destination}"


def _get_or_create_logger(destination: str = _DEFAULT_DESTINATION) -> logging.Logger:
    handler, name = _get_logging_handler(destination)
    logger = logging.getLogger(f"torchrec_b200-{name}")
    logger.setLevel(logging.DEBUG)
    if not any(h is handler for h in logger.handlers):
        handler.setFormatter(logging.Formatter("%(asctime)s %(filename)s:%(lineno)s %(levelname)s p:%(processName)s t:%(threadName)s: %(message)s"))
        logger.propagate = False
        logger.addHandler(handler)
    return logger


def _get_msg_dict(func_name: str, **kwargs: Any) -> Dict[str, Any]:
    msg = {"func_name": func_name}
    if dist.is_available() and dist.is_initialized():
        group = kwargs.get("group") or kwargs.get("process_group")
        msg.update({"group": f"{group}", "world_size": f"{dist.get_world_size(group)}", "rank": f"{dist.get_rank(group)}"})
    return msg
