"""Turning a sharded training checkpoint into plain tensors for serving (``torchrec/inference/state_dict_transform.py``)."""
from __future__ import annotations

from typing import Dict, List, Optional, Union

import torch
import torch.distributed as dist

from torchrec_b200.distributed.types import ShardedTensor


def state_dict_gather(src: Dict[str, Union[torch.Tensor, ShardedTensor]], dst: Dict[str, torch.Tensor]) -> None:
    """Collective: gather every sharded entry of ``src`` into the full tensor ``dst[key]`` on rank 0; plain tensors are copied."""
    for key, dst_tensor in dst.items():
        src_tensor = src[key]
        if isinstance(src_tensor, ShardedTensor):
            src_tensor.gather(out=dst_tensor if dist.get_rank() == 0 else None)
        else:
            dst_tensor.copy_(src_tensor)


def state_dict_all_gather_keys(state_dict: Dict[str, Union[torch.Tensor, ShardedTensor]], pg: Optional[dist.ProcessGroup] = None) -> List[str]:
    """Union of the keys of all ranks (a rank need not hold every table)."""
    names = list(state_dict.keys())
    all_names: List[Optional[List[str]]] = [None] * dist.get_world_size(pg)
    dist.all_gather_object(all_names, names, pg)
    deduped = {n: None for group in all_names for n in (group or [])}
    return sorted(deduped.keys())


def state_dict_to_device(state_dict: Dict[str, Union[torch.Tensor, ShardedTensor]], pg: Optional[dist.ProcessGroup], device: torch.device) -> Dict[str, Union[torch.Tensor, ShardedTensor]]:
    """Move every tensor (and the local shards of sharded ones) to ``device`` keeping the sharding metadata."""
    from torch.distributed._shard.sharded_tensor import Shard

    ret: Dict[str, Union[torch.Tensor, ShardedTensor]] = {}
    all_keys = state_dict_all_gather_keys(state_dict, pg)
    for key in all_keys:
        if key not in state_dict:
            continue
        t = state_dict[key]
        if isinstance(t, ShardedTensor):
            shards = [Shard(s.tensor.to(device), s.metadata) for s in t.local_shards()]
            ret[key] = ShardedTensor._init_from_local_shards_and_global_metadata(shards, t.metadata(), process_group=pg)
        else:
            ret[key] = t.to(device)
    return ret
