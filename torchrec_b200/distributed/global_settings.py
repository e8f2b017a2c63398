"""Process-wide switches of the sharding runtime (``torchrec/distributed/global_settings.py``).

``propogate_device`` (spelling kept for compatibility): sharders place tables on the device they are given instead of the
process's default accelerator.  ``TORCHREC_CONSTRUCT_SHARDED_TENSOR_FROM_METADATA=1``: build checkpoint tensors from plan
metadata without a collective.
"""
from __future__ import annotations

import os
from dataclasses import dataclass


@dataclass
class _Settings:
    propogate_device: bool = False


_settings = _Settings()
TORCHREC_CONSTRUCT_SHARDED_TENSOR_FROM_METADATA_ENV = "TORCHREC_CONSTRUCT_SHARDED_TENSOR_FROM_METADATA"


def set_propogate_device(val: bool) -> None:
    _settings.propogate_device = bool(val)


def get_propogate_device() -> bool:
    return _settings.propogate_device


def construct_sharded_tensor_from_metadata_enabled() -> bool:
    return os.environ.get(TORCHREC_CONSTRUCT_SHARDED_TENSOR_FROM_METADATA_ENV, "0") == "1"
