"""Helpers for tests: free ports, seeding, multi-process runners (cf. ``torchrec/test_utils/__init__.py``)."""
from __future__ import annotations

import os
import random
import socket
import time
from contextlib import closing
from typing import Optional

import numpy as np
import torch


def get_free_port() -> int:
    with closing(socket.socket(socket.AF_INET, socket.SOCK_STREAM)) as s:
        s.bind(("127.0.0.1", 0))
        s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        return s.getsockname()[1]


def seed_and_log(seed: Optional[int] = None) -> int:
    if seed is None:
        seed = int(time.time()) % 2 ** 31
    print(f"seed: {seed}")
    torch.manual_seed(seed)
    np.random.seed(seed)
    random.seed(seed)
    return seed


def init_distributed_single_host(rank: int, world_size: int, backend: str, local_size: Optional[int] = None):
    os.environ["LOCAL_WORLD_SIZE"] = str(local_size if local_size else world_size)
    os.environ["LOCAL_RANK"] = str(rank % local_size if local_size else rank)
    import torch.distributed as dist

    dist.init_process_group(rank=rank, world_size=world_size, backend=backend)
    return dist.group.WORLD
