"""Process-wide switches (``torchrec/distributed/global_settings.py``)."""
import os

PROPOGATE_DEVICE: bool = False
TORCHREC_CONSTRUCT_SHARDED_TENSOR_FROM_METADATA_ENV = "TORCHREC_CONSTRUCT_SHARDED_TENSOR_FROM_METADATA"


def set_propogate_device(val: bool) -> None:
    global PROPOGATE_DEVICE
    PROPOGATE_DEVICE = val


def get_propogate_device() -> bool:
    return PROPOGATE_DEVICE


def construct_sharded_tensor_from_metadata_enabled() -> bool:
    return os.environ.get(TORCHREC_CONSTRUCT_SHARDED_TENSOR_FROM_METADATA_ENV, "0") == "1"
