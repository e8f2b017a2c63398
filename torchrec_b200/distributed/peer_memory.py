"""Peer-mapped device buffers and a device-side barrier for one process group on one node.

Every rank allocates a buffer, hands an inter-process handle of it to its peers and maps theirs, so a kernel on
this GPU can store into / load from the buffer of any rank over NVLink.  This is what the fused embedding lookup
uses to write pooled rows straight into the [B_local, D] buffer of the rank that owns the sample (and to pull
gradient rows back), instead of materialising a send buffer and calling an all-to-all.

The reference framework has no such layer; its exchanges are library collectives
(``torchrec/distributed/comm_ops.py:574-1073``).

Only used when every rank of the group sits on the same node and peer access works; ``PeerGroup.get`` agrees on that
across the group (one all-reduce) so that either all ranks use the fused path or none does.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

_GROUPS: Dict[Tuple[int, int], Optional["PeerGroup"]] = {}


def peer_exchange_enabled() -> bool:
    return os.environ.get("TRB200_PEER_EXCHANGE", "1") != "0"


class PeerGroup:
    """Shares buffers with the ranks of ``pg`` and runs the bounded device-side barrier."""

    def __init__(self, pg: dist.ProcessGroup, device: torch.device) -> None:
        self.pg = pg
        self.device = device
        self.world = dist.get_world_size(pg)
        self.rank = dist.get_rank(pg)
        self._keepalive: List[torch.Tensor] = []
        self._epoch = 0
        self.ok = True  # local view; ``get`` combines it over the group
        self.error: Optional[str] = None
        self.err = torch.zeros(1, dtype=torch.int32, device=device)
        # flags[0:world]: barrier arrivals; flags[world:2*world]: a pattern the peers read back to verify their mapping
        self.flags, self.flag_ptrs = self.alloc_shared((2 * self.world,), torch.int32)
        self.flags[self.world:] = 1000 + self.rank
        torch.cuda.synchronize(device)
        dist.barrier(group=pg)
        try:
            for r, ptr in enumerate(self.flag_ptrs):
                if r == self.rank or not self.ok:
                    continue
                got = torch.ops.trb200.peer_read(ptr + 4 * self.world, 4 * self.world, device).view(torch.int32)
                if not bool((got == 1000 + r).all()):
                    self.ok = False
                    self.error = f"rank {r}'s buffer reads back wrong through the peer mapping"
        except Exception as e:
            self.ok = False
            self.error = f"reading a peer buffer failed: {type(e).__name__}: {e}"
        dist.barrier(group=pg)

    # -- sharing ------------------------------------------------------------------------------------------
    def alloc_shared(self, shape, dtype: torch.dtype) -> Tuple[torch.Tensor, List[int]]:
        """Collective.  Allocates a zeroed buffer of ``shape`` on every rank and maps all of them everywhere.  Returns
        this rank's buffer and the device addresses of all ranks' buffers (index = rank) valid for kernels here."""
        numel = 1
        for d in shape:
            numel *= int(d)
        nbytes = max(numel, 1) * torch.empty(0, dtype=dtype).element_size()
        raw = None
        handle = None
        try:
            raw = torch.ops.trb200.peer_alloc(nbytes, self.device)
            handle = torch.ops.trb200.peer_handle(raw)
        except Exception as e:
            self.ok = False
            self.error = f"allocating a shareable buffer failed: {type(e).__name__}: {e}"
        gathered: List[Optional[torch.Tensor]] = [None] * self.world
        dist.all_gather_object(gathered, handle, group=self.pg)
        if raw is None:
            raw = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
        local = raw[: numel * torch.empty(0, dtype=dtype).element_size()].view(dtype).view(*shape)
        ptrs: List[int] = []
        for r, h in enumerate(gathered):
            if r == self.rank:
                ptrs.append(local.data_ptr())
                continue
            try:
                if h is None:
                    raise RuntimeError("the peer has no handle")
                ptrs.append(int(torch.ops.trb200.peer_open(h, self.device)))
            except Exception as e:
                self.ok = False
                self.error = f"mapping rank {r}'s buffer failed: {type(e).__name__}: {e}"
                ptrs.append(local.data_ptr())
        self._keepalive.append(raw)
        return local, ptrs

    # -- barrier ------------------------------------------------------------------------------------------
    def barrier(self) -> None:
        """Enqueue the device-side barrier on the current stream (host does not wait)."""
        self._epoch += 1
        torch.ops.trb200.peer_barrier(self.flag_ptrs, self.rank, self._epoch, self.err)

    def check_error(self) -> None:
        """Host read of the barrier error word (synchronises); raises if a peer never arrived."""
        v = int(self.err.item())
        if v != 0:
            self.err.zero_()
            raise RuntimeError(f"peer barrier timed out waiting for rank {v - 100}")

    # -- construction -------------------------------------------------------------------------------------
    @staticmethod
    def get(pg: Optional[dist.ProcessGroup], device: Optional[torch.device]) -> Optional["PeerGroup"]:
        """The group's ``PeerGroup`` or None when the fused exchange cannot be used (decided collectively)."""
        if pg is None or device is None or device.type != "cuda" or not peer_exchange_enabled():
            return None
        if not dist.is_initialized() or dist.get_backend(pg) != "nccl" or dist.get_world_size(pg) < 2:
            return None
        key = (id(pg), device.index if device.index is not None else torch.cuda.current_device())
        if key in _GROUPS:
            return _GROUPS[key]
        world = dist.get_world_size(pg)
        ok = 1
        try:
            from torchrec_b200.ops import _ext

            local_world = int(os.environ.get("LOCAL_WORLD_SIZE", world))
            if not _ext.has_cuda_ext() or world > 16 or local_world < world or torch.cuda.device_count() < world:
                ok = 0
            else:
                me = key[1]
                for d in range(torch.cuda.device_count()):
                    if d != me and not torch.cuda.can_device_access_peer(me, d):
                        ok = 0
        except Exception:
            ok = 0
        flag = torch.tensor([ok], dtype=torch.int32, device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=pg)
        group: Optional[PeerGroup] = None
        if int(flag.item()) == 1:
            group = PeerGroup(pg, device)  # its collectives run on every rank even if a local step fails
            flag = torch.tensor([1 if group.ok else 0], dtype=torch.int32, device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=pg)
            if int(flag.item()) != 1:
                import warnings

                warnings.warn(f"fused peer exchange disabled, falling back to library collectives: {group.error or 'a peer reported a failure'}")
                group = None
        _GROUPS[key] = group
        return group
