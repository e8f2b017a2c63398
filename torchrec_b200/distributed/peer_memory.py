"""Peer-mapped device buffers and device-side flag synchronisation for the ranks of one node.

Every rank allocates a buffer, hands an inter-process handle of it to its peers and maps theirs, so a kernel on
this GPU can store into / load from the buffer of any rank over NVLink.  The fused sparse engine
(``fused_sparse_engine.py``) uses this to deliver ids, pooled rows and gradient rows without a collective call, and
the dense data-parallel wrapper (``peer_data_parallel.py``) to all-reduce gradients.

Synchronisation is by flags in the same kind of memory (``FlagSet``): epochs are counted on the device, so the
launches can be captured once in a CUDA graph and replayed.  Every wait is bounded (``TRB200_PEER_WAIT_S`` seconds,
default 30); a wait that runs out stores a code in the group's error word, results of that step are poisoned with
NaN by the consuming kernels, and ``poll_error`` / ``check_error`` raise on the host.

Three flavours share one interface (``rank``, ``world``, ``alloc_shared``, ``free_shared``, ``new_flags``):

* ``PeerGroup``       real ranks, one process per GPU, buffers shared through CUDA IPC handles;
* ``SoloPeerGroup``   world size 1: plain local buffers, the same kernels run unchanged;
* ``EmulatedPeerGroup`` several *virtual* ranks on ONE GPU for tests: buffers are local, and the caller runs every
  virtual rank's phase k before any rank's phase k+1, so no kernel ever waits for a later launch.

The reference framework has no such layer; its exchanges are library collectives
(``torchrec/distributed/comm_ops.py:574-1073``).
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

_GROUPS: Dict[Tuple[int, int], Optional["PeerGroup"]] = {}
_SM_HZ = 1.9e9  # wait limits are given to kernels in SM clock cycles


def peer_exchange_enabled() -> bool:
    return os.environ.get("TRB200_PEER_EXCHANGE", "1") != "0"


def default_wait_cycles() -> int:
    return int(float(os.environ.get("TRB200_PEER_WAIT_S", "30")) * _SM_HZ)


_ERR_TEXT = {
    1: "an id lies outside its table",
    300: "the receive buffer of the fused input distribution is too small for this batch (raise TRB200_DIST_SLACK)",
}


def describe_error(code: int) -> str:
    if code in _ERR_TEXT:
        return _ERR_TEXT[code]
    for base, what in ((100, "a peer barrier"), (200, "the split sizes of the input distribution"), (220, "the ids of the input distribution"),
                       (250, "(batch sizes differ between ranks)"), (400, "the gradient all-reduce")):
        if base <= code < base + 16:
            return f"timed out waiting for rank {code - base} in {what}" if base != 250 else f"rank {code - base} runs a different per-rank batch size"
    return f"device status {code}"


_ALL: List["_PeerBase"] = []


def poll_all() -> None:
    """``poll_error`` on every peer layer of this process (training loops call it once per step)."""
    for g in _ALL:
        g.poll_error()


def check_all() -> None:
    """``check_error`` on every peer layer of this process (synchronises)."""
    for g in _ALL:
        g.check_error()


class FlagSet:
    """``nslots`` synchronisation points: peer-mapped flags ``[nslots, world]`` plus local device-side epoch counters."""

    def __init__(self, group: "_PeerBase", nslots: int) -> None:
        self.group = group
        self.nslots = nslots
        self.local, self.ptrs = group.alloc_shared((nslots * group.world,), torch.int32)
        self.epochs = torch.zeros(nslots, dtype=torch.int32, device=group.device)

    def sync(self, slot: int, signal: bool = True, wait: bool = True) -> None:
        """Enqueue on the current stream: raise this rank's flag of ``slot`` on every peer and / or wait for all peers."""
        g = self.group
        torch.ops.trb200.peer_sync(self.ptrs, g.rank, slot, self.epochs, signal, wait, g.wait_cycles, g.err)

    def signal(self, slot: int) -> None:
        self.sync(slot, True, False)

    def wait(self, slot: int) -> None:
        self.sync(slot, False, True)


class _PeerBase:
    rank: int
    world: int
    device: torch.device

    def _init_common(self, device: torch.device) -> None:
        if device.type == "cuda":
            # every method of a peer group launches kernels of the CUDA library: load it here (and fail loudly without it), so that a
            # group can be the first thing a process builds
            from torchrec_b200.ops import _ext

            _ext.require_cuda_ext("peer group")
        self.device = device
        self.err = torch.zeros(1, dtype=torch.int32, device=device)
        self.wait_cycles = default_wait_cycles()
        self._err_host = torch.zeros(1, dtype=torch.int32).pin_memory() if device.type == "cuda" else torch.zeros(1, dtype=torch.int32)
        self._err_event: Optional[torch.cuda.Event] = None
        if device.type == "cuda":
            _ALL.append(self)

    def new_flags(self, nslots: int) -> FlagSet:
        return FlagSet(self, nslots)

    # -- error word ---------------------------------------------------------------------------------------
    def check_error(self) -> None:
        """Host read of the error word (synchronises); raises if a bounded wait ran out or a size check failed."""
        v = int(self.err.item())
        if v != 0:
            self.err.zero_()
            raise RuntimeError(f"fused exchange failed on rank {self.rank}: {describe_error(v)}")

    def poll_error(self) -> None:
        """Non-blocking form for the training loop: starts an asynchronous copy of the error word and inspects the copy
        started by the previous call once it has landed.  Never call it while the current stream is being captured."""
        if self._err_event is not None and self._err_event.query():
            v = int(self._err_host[0])
            self._err_event = None
            if v != 0:
                self.err.zero_()
                raise RuntimeError(f"fused exchange failed on rank {self.rank}: {describe_error(v)}")
        if self._err_event is None:
            self._err_host.copy_(self.err, non_blocking=True)
            self._err_event = torch.cuda.Event()
            self._err_event.record()

    def alloc_shared(self, shape, dtype: torch.dtype) -> Tuple[torch.Tensor, List[int]]:
        raise NotImplementedError

    def free_shared(self, local: torch.Tensor, ptrs: List[int]) -> None:
        raise NotImplementedError


def _nbytes(shape, dtype: torch.dtype) -> Tuple[int, int]:
    numel = 1
    for d in shape:
        numel *= int(d)
    return numel, max(numel, 1) * torch.empty(0, dtype=dtype).element_size()


class SoloPeerGroup(_PeerBase):
    """World size 1 on a CUDA device: the 'peers' are this rank itself."""

    def __init__(self, device: torch.device) -> None:
        self.rank, self.world = 0, 1
        self._init_common(device)

    def alloc_shared(self, shape, dtype):
        t = torch.zeros(*shape, dtype=dtype, device=self.device)
        return t, [t.data_ptr()]

    def free_shared(self, local, ptrs) -> None:
        return None


class EmulatedPeerGroup:
    """``world`` virtual ranks on one GPU (tests).  ``view(r)`` is rank r's handle; the k-th ``alloc_shared`` call of every
    view returns the k-th shared allocation, like the collective allocation of real ranks."""

    def __init__(self, world: int, device: torch.device, wait_cycles: Optional[int] = None) -> None:
        self.world = world
        self.device = device
        self._allocs: List[List[torch.Tensor]] = []
        self._views = [_EmulatedView(self, r) for r in range(world)]
        if wait_cycles is not None:
            for v in self._views:
                v.wait_cycles = wait_cycles

    def view(self, rank: int) -> "_EmulatedView":
        return self._views[rank]

    def _get(self, k: int, shape, dtype) -> List[torch.Tensor]:
        if k == len(self._allocs):
            self._allocs.append([torch.zeros(*shape, dtype=dtype, device=self.device) for _ in range(self.world)])
        bufs = self._allocs[k]
        assert tuple(bufs[0].shape) == tuple(int(s) for s in shape) and bufs[0].dtype == dtype, "virtual ranks must allocate alike"
        return bufs


class _EmulatedView(_PeerBase):
    def __init__(self, parent: EmulatedPeerGroup, rank: int) -> None:
        self.parent = parent
        self.rank, self.world = rank, parent.world
        self._k = 0
        self._init_common(parent.device)

    def alloc_shared(self, shape, dtype):
        bufs = self.parent._get(self._k, shape, dtype)
        self._k += 1
        return bufs[self.rank], [b.data_ptr() for b in bufs]

    def free_shared(self, local, ptrs) -> None:
        return None


class PeerGroup(_PeerBase):
    """Shares buffers with the ranks of ``pg`` (one process per GPU, all on one node)."""

    def __init__(self, pg: dist.ProcessGroup, device: torch.device) -> None:
        self.pg = pg
        self.world = dist.get_world_size(pg)
        self.rank = dist.get_rank(pg)
        self._init_common(device)
        self._keepalive: Dict[int, torch.Tensor] = {}
        self.ok = True  # local view; ``get`` combines it over the group
        self.error: Optional[str] = None
        # a pattern the peers read back through their mapping before any kernel uses one
        probe, probe_ptrs = self.alloc_shared((self.world,), torch.int32)
        probe[:] = 1000 + self.rank
        torch.cuda.synchronize(device)
        dist.barrier(group=pg)
        try:
            for r, ptr in enumerate(probe_ptrs):
                if r == self.rank or not self.ok:
                    continue
                got = torch.ops.trb200.peer_read(ptr, 4 * self.world, device).view(torch.int32)
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
        numel, nbytes = _nbytes(shape, dtype)
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
        self._keepalive[local.data_ptr()] = raw
        return local, ptrs

    def free_shared(self, local: torch.Tensor, ptrs: List[int]) -> None:
        """Collective.  Unmaps the peers' buffers of one ``alloc_shared`` call and releases this rank's own, after every
        rank has drained its device work."""
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.pg)
        for r, ptr in enumerate(ptrs):
            if r != self.rank and ptr != local.data_ptr():
                try:
                    torch.ops.trb200.peer_close(ptr, self.device)
                except Exception:
                    pass
        dist.barrier(group=self.pg)
        self._keepalive.pop(local.data_ptr(), None)

    # -- construction -------------------------------------------------------------------------------------
    @staticmethod
    def get(pg: Optional[dist.ProcessGroup], device: Optional[torch.device]) -> Optional[_PeerBase]:
        """The group's peer layer, or None when the fused exchange cannot be used (decided collectively).  A group of
        one rank on a CUDA device gets a ``SoloPeerGroup``."""
        if device is None or device.type != "cuda" or not peer_exchange_enabled():
            return None
        from torchrec_b200.ops import _ext

        if not _ext.has_cuda_ext():
            return None
        world = dist.get_world_size(pg) if (pg is not None and dist.is_initialized()) else 1
        key = (id(pg), device.index if device.index is not None else torch.cuda.current_device())
        if key in _GROUPS:
            return _GROUPS[key]
        if world == 1:
            _GROUPS[key] = SoloPeerGroup(device)
            return _GROUPS[key]
        if dist.get_backend(pg) != "nccl":
            return None
        ok = 1
        try:
            local_world = int(os.environ.get("LOCAL_WORLD_SIZE", world))
            if world > 16 or local_world < world or torch.cuda.device_count() < world:
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
