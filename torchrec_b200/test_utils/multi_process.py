"""Run a function as ``world_size`` ranks on one host (cf. ``torchrec/distributed/test_utils/multi_process.py``).

Ranks use ``cuda:{rank}`` when enough GPUs exist and the backend is ``nccl``, otherwise the CPU with
``gloo``.  Rendezvous is on 127.0.0.1 with a free port.  Every rank must exit with code 0.
"""
from __future__ import annotations

import multiprocessing
import os
import traceback
from typing import Any, Callable, Dict, Optional

import torch
import torch.distributed as dist

from torchrec_b200.test_utils import get_free_port


class MultiProcessContext:
    def __init__(self, rank: int, world_size: int, backend: str = "gloo", local_size: Optional[int] = None, use_deterministic_algorithms: bool = False, timeout_s: int = 120) -> None:
        self.rank = rank
        self.world_size = world_size
        self.backend = backend
        self.local_size = local_size
        self.timeout_s = timeout_s
        if torch.cuda.is_available() and world_size <= torch.cuda.device_count() and backend == "nccl":
            self.device = torch.device(f"cuda:{rank}")
            torch.cuda.set_device(self.device)
        else:
            self.device = torch.device("cpu")
        self.pg: Optional[dist.ProcessGroup] = None

    def __enter__(self) -> "MultiProcessContext":
        import datetime

        os.environ["LOCAL_WORLD_SIZE"] = str(self.local_size if self.local_size else self.world_size)
        os.environ["LOCAL_RANK"] = str(self.rank % self.local_size if self.local_size else self.rank)
        dist.init_process_group(rank=self.rank, world_size=self.world_size, backend=self.backend, timeout=datetime.timedelta(seconds=self.timeout_s))
        self.pg = dist.group.WORLD
        return self

    def __exit__(self, exc_type, exc_instance, tb) -> None:
        from torchrec_b200.distributed.comm import reset_node_process_groups

        reset_node_process_groups()
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:
                pass


def _wrapper(fn: Callable, rank: int, world_size: int, port: int, kwargs: Dict[str, Any], err_q) -> None:
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["RANK"] = str(rank)
    os.environ["WORLD_SIZE"] = str(world_size)
    os.environ.setdefault("GLOO_DEVICE_TRANSPORT", "TCP")
    os.environ.setdefault("GLOO_SOCKET_IFNAME", "lo")
    os.environ.setdefault("NCCL_SOCKET_IFNAME", "lo")
    torch.set_num_threads(1)
    try:
        fn(rank, world_size, **kwargs)
    except BaseException:
        err_q.put((rank, traceback.format_exc()))
        raise


def run_multi_process(fn: Callable[..., None], world_size: int = 2, timeout_s: int = 300, **kwargs) -> None:
    """Spawn ``world_size`` processes running ``fn(rank, world_size, **kwargs)`` and assert all succeed."""
    ctx = multiprocessing.get_context("spawn")
    port = get_free_port()
    err_q = ctx.Queue()
    procs = []
    for rank in range(world_size):
        p = ctx.Process(target=_wrapper, args=(fn, rank, world_size, port, kwargs, err_q), name=f"rank{rank}")
        p.start()
        procs.append(p)
    for p in procs:
        p.join(timeout_s)
    errors = []
    while not err_q.empty():
        errors.append(err_q.get())
    for p in procs:
        if p.is_alive():
            p.kill()
            errors.append((p.name, "timed out"))
    bad = [p.name for p in procs if p.exitcode != 0]
    assert not bad and not errors, "ranks failed: " + "\n".join(f"[{r}] {tb}" for r, tb in errors) + f" exit codes: {[p.exitcode for p in procs]}"
