"""Data parallelism of the dense (unsharded) part of a model over peer-mapped memory.

``PeerDataParallelWrapper`` is a ``DataParallelWrapper`` for ``DistributedModelParallel``.  Instead of wrapping the
model in ``DistributedDataParallel`` it

* broadcasts rank 0's dense parameters once,
* moves them into one flat fp32 buffer with a flat gradient buffer that lives in memory every rank of the node has
  mapped (``FlatParamBuffer``), and
* at the end of every backward pass averages the flat gradient in place with ONE kernel (``peer_allreduce``: reduce-
  scatter + all-gather by plain peer loads and stores, deterministic summation order), followed by a bounded wait.

No bucket bookkeeping runs on the host and nothing in it depends on host state, so the whole step can be captured in a
CUDA graph.  When the ranks cannot map each other's memory (several nodes, no peer access, CPU) the wrapper falls back
to ``DefaultDataParallelWrapper``.

Reference: ``torchrec/distributed/model_parallel.py:83-145`` (DDP with 25 MB NCCL buckets).
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist
from torch import nn

from torchrec_b200.distributed.model_parallel import DataParallelWrapper, DefaultDataParallelWrapper, DistributedModelParallel
from torchrec_b200.distributed.peer_memory import PeerGroup, _PeerBase
from torchrec_b200.optim.fused_dense import FlatParamBuffer

SLOT_AR_IN, SLOT_AR_OUT = 0, 1


class PeerGradSync:
    """Flat dense gradients of one model replica and their in-place average over the ranks of ``peer``."""

    def __init__(self, params: List[nn.Parameter], peer: _PeerBase) -> None:
        self.peer = peer
        self.world = peer.world
        self._grad_ptrs: List[int] = []

        def alloc(n: int) -> torch.Tensor:
            local, ptrs = peer.alloc_shared((n,), torch.float32)
            self._grad_ptrs = ptrs
            return local

        self.buffer = FlatParamBuffer(params, grad_alloc=alloc)
        self.flags = peer.new_flags(2)
        self.counter = torch.zeros(1, dtype=torch.int32, device=peer.device)
        self._armed = False
        self.enabled = True
        for p in self.buffer.params:
            p.register_post_accumulate_grad_hook(self._on_grad)
        self.buffer.on_direct_write = self._on_grad  # gradients written by kernels bypass the accumulation hooks

    def _on_grad(self, _p: Optional[torch.Tensor] = None) -> None:
        if not self._armed and self.enabled:
            self._armed = True
            torch.autograd.Variable._execution_engine.queue_callback(self._finish_backward)

    def _finish_backward(self) -> None:
        self._armed = False
        self.all_reduce()

    def all_reduce(self, signal_inside: bool = True) -> None:
        """Average the flat gradient over all ranks, in place, on the current stream."""
        if self.world == 1:
            return
        b = self.buffer
        if not torch.cuda.is_current_stream_capturing():
            b.attach_grads()
        p = self.peer
        torch.ops.trb200.peer_allreduce(self._grad_ptrs, b.total, 1.0 / self.world, self.flags.ptrs, p.rank, SLOT_AR_IN, SLOT_AR_OUT,
                                        self.flags.epochs, self.counter, signal_inside, p.wait_cycles, p.err)
        self.flags.wait(SLOT_AR_OUT)


class PeerDataParallelWrapper(DataParallelWrapper):
    """See the module docstring.  ``fallback`` wraps the model when the peer layer is unavailable."""

    def __init__(self, fallback=None, params_to_ignore: Optional[List[str]] = None) -> None:
        self._fallback = fallback
        self._ignore = set(params_to_ignore or [])

    def wrap(self, dmp, env, device: torch.device) -> None:
        if getattr(dmp, "_peer_grad_sync", None) is not None:
            return
        pg = env.process_group
        peer = PeerGroup.get(pg, device) if device.type == "cuda" else None
        if peer is None:
            (self._fallback or DefaultDataParallelWrapper()).wrap(dmp, env, device)
            return
        sharded = set(DistributedModelParallel._sharded_parameter_names(dmp._dmp_wrapped_module)) | self._ignore
        params = [p for n, p in dmp._dmp_wrapped_module.named_parameters() if p.requires_grad and n not in sharded and p.dtype == torch.float32
                  and not getattr(p, "_in_backward_optimizers", None)]
        if not params:
            return
        if peer.world > 1:
            with torch.no_grad():
                for p in params:
                    dist.broadcast(p.data, src=dist.get_global_rank(pg, 0) if pg is not None else 0, group=pg)
        dmp._peer_grad_sync = PeerGradSync(params, peer)
