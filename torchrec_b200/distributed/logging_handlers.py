"""Registry of log handlers by destination name; deployments add their own (``torchrec/distributed/logging_handlers.py:12``)."""
import logging
from typing import Dict

_log_handlers: Dict[str, logging.Handler] = {"default": logging.NullHandler()}
