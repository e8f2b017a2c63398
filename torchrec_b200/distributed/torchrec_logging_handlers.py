"""Registers the library's own log destination (a no-op handler until a deployment replaces it) in the handler registry
(``torchrec/distributed/torchrec_logging_handlers.py``)."""
import logging

from torchrec_b200.distributed.logging_handlers import _log_handlers

TORCHREC_LOGGER_NAME = "torchrec"

_log_handlers.setdefault(TORCHREC_LOGGER_NAME, logging.NullHandler())
