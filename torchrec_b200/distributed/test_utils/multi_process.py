"""Spawned-process test harness (``torchrec/distributed/test_utils/multi_process.py``)."""
from torchrec_b200.test_utils.multi_process import MultiProcessContext, run_multi_process  # noqa: F401
