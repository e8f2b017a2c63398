"""Run a function on one rank and give every rank its result (cf. ``torchrec/distributed/collective_utils.py``)."""
from __future__ import annotations

from typing import Callable, TypeVar

import torch.distributed as dist

T = TypeVar("T")


def is_leader(pg, leader_rank: int = 0) -> bool:
    if pg is None:
        return leader_rank == 0
    return pg.rank() == leader_rank


def invoke_on_rank_and_broadcast_result(pg: dist.ProcessGroup, rank: int, func: Callable[..., T], *args, **kwargs) -> T:
    """``func`` runs on ``rank`` only; its (picklable) result is broadcast to the group.
    An exception raised by ``func`` is re-raised on every rank."""
    res, exc = None, None
    if pg.rank() == rank:
        try:
            res = func(*args, **kwargs)
        except Exception as e:  # noqa: BLE001 - forwarded to all ranks
            exc = e
    object_list = [(res, exc)]
    if pg.size() > 1:
        dist.broadcast_object_list(object_list, dist.get_global_rank(pg, rank) if hasattr(dist, "get_global_rank") else rank, group=pg)
    res, exc = object_list[0]
    if exc is not None:
        raise exc
    return res


def run_on_leader(pg: dist.ProcessGroup, rank: int):
    def callable(func):
        def wrapped(*args, **kwargs):
            return invoke_on_rank_and_broadcast_result(pg, rank, func, *args, **kwargs)
        return wrapped
    return callable
