"""Process-group helpers (cf. ``torchrec/distributed/comm.py:38-276``).

Local (per-node) size and rank come from the launcher's environment; intra-node and
cross-node sub-groups are built for the hierarchical shardings (TWRW / GRID) and for 2D
parallelism.  On a single NVSwitch box every rank is "local", so the intra-node group is the
world and the cross-node group has one member.
"""
from __future__ import annotations

import logging
import os
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

logger: logging.Logger = logging.getLogger(__name__)

_INTRA_PG: Optional[dist.ProcessGroup] = None
_CROSS_PG: Optional[dist.ProcessGroup] = None
_NODE_GROUP_SIZE_2D: Optional[int] = None  # ranks per node inside a sharding group, set when the 2D node groups are built


def _env2int(env_list: List[str], default: int = -1) -> int:
    for e in env_list:
        val = int(os.environ.get(e, -1))
        if val >= 0:
            return val
    return default


def get_local_size(world_size: Optional[int] = None) -> int:
    if world_size is None:
        world_size = dist.get_world_size()
    local_size = _env2int(["LOCAL_WORLD_SIZE", "MPI_LOCALNRANKS", "OMPI_COMM_WORLD_LOCAL_SIZE", "MV2_COMM_WORLD_LOCAL_SIZE"], 8)
    if local_size == -1 or world_size % local_size != 0:
        logging.warning("Could not determine LOCAL_WORLD_SIZE from environment, falling back to WORLD_SIZE.")
        local_size = world_size
    return local_size


def get_node_group_size(world_size: Optional[int] = None) -> int:
    """Ranks per node as the sharding group of a 2D-parallel job sees them (recorded by ``intra_and_cross_node_pg_2D``); the plain
    local size when no 2D groups were built."""
    if _NODE_GROUP_SIZE_2D is None:
        return get_local_size(world_size)
    return _NODE_GROUP_SIZE_2D


def get_local_rank(world_size: Optional[int] = None, rank: Optional[int] = None) -> int:
    my_local_rank = _env2int(["LOCAL_RANK", "MPI_LOCALRANKID", "OMPI_COMM_WORLD_LOCAL_RANK", "MV2_COMM_WORLD_LOCAL_RANK"], -1)
    local_size = get_local_size(world_size)
    if my_local_rank == -1 or my_local_rank >= local_size:
        logging.warning("Could not determine LOCAL_RANK from environment, falling back to GLOBAL_RANK % LOCAL_SIZE.")
        if rank is None:
            rank = dist.get_rank()
        my_local_rank = rank % local_size
    return my_local_rank


def get_group_rank(world_size: Optional[int] = None, rank: Optional[int] = None) -> int:
    """Index of the node ("group") this rank belongs to."""
    if rank is None:
        rank = dist.get_rank()
    return rank // get_local_size(world_size)


def get_num_groups(world_size: Optional[int] = None) -> int:
    if world_size is None:
        world_size = dist.get_world_size()
    return world_size // get_local_size(world_size)


def intra_and_cross_node_pg(
    device: Optional[torch.device] = None, backend: Optional[str] = None,
) -> Tuple[Optional[dist.ProcessGroup], Optional[dist.ProcessGroup]]:
    """Sub-groups of the ranks on this node and of the ranks with the same local index on all nodes."""
    global _INTRA_PG, _CROSS_PG
    world, me = dist.get_world_size(), dist.get_rank()
    per_node = get_local_size(world)
    nodes = get_num_groups(world)
    backend = backend or dist.get_backend()

    def make_family(groups: List[List[int]]) -> Optional[dist.ProcessGroup]:
        # group creation is collective: every rank creates every group and keeps the one it is a member of
        mine = None
        for ranks in groups:
            pg = dist.new_group(backend=backend, ranks=ranks)
            if me in ranks:
                mine = pg
        dist.barrier()
        return mine

    if _INTRA_PG is None:
        _INTRA_PG = make_family([list(range(n * per_node, (n + 1) * per_node)) for n in range(nodes)])
    if _CROSS_PG is None:
        _CROSS_PG = make_family([list(range(i, world, per_node)) for i in range(per_node)])
    return _INTRA_PG, _CROSS_PG


def reset_node_process_groups() -> None:
    global _INTRA_PG, _CROSS_PG, _NODE_GROUP_SIZE_2D
    _INTRA_PG = None
    _CROSS_PG = None
    _NODE_GROUP_SIZE_2D = None


def intra_and_cross_node_pg_2D(env, device: Optional[torch.device] = None):
    """Intra/cross node groups inside the sharding group of a 2D environment."""
    backend = dist.get_backend(env.sharding_pg)
    my_rank = dist.get_rank()
    sharding_group_size = dist.get_world_size(env.sharding_pg)
    world_size = dist.get_world_size()
    local_size = env.node_group_size if env.node_group_size else get_local_size(world_size)
    global _NODE_GROUP_SIZE_2D
    _NODE_GROUP_SIZE_2D = local_size
    num_sharding_groups = world_size // sharding_group_size
    step = 1 if env.use_inter_host_allreduce else num_sharding_groups
    intra_pg = cross_pg = None
    for g in range(num_sharding_groups):
        ranks = (
            list(range(g * sharding_group_size, (g + 1) * sharding_group_size))
            if env.use_inter_host_allreduce else list(range(g, world_size, step))
        )
        nodes = [ranks[i: i + local_size] for i in range(0, len(ranks), local_size)]
        for node in nodes:
            pg = dist.new_group(ranks=node, backend=backend)
            if my_rank in node:
                intra_pg = pg
        for l in range(local_size):
            peers = [node[l] for node in nodes if l < len(node)]
            pg = dist.new_group(ranks=peers, backend=backend)
            if my_rank in peers:
                cross_pg = pg
    dist.barrier()
    return intra_pg, cross_pg
