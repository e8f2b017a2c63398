"""Fused sequence engine: a sharded ``EmbeddingCollection`` step (one row per id, no pooling) over peer-mapped memory.

The classic path runs, per sharding type, a split-size all-to-all with a host read, one all-to-all per KJT tensor, the
lookup, a sequence all-to-all whose split sizes come from the forward lengths, and for row-wise tables an extra gather that
undoes the bucketization (``torchrec/distributed/dist_data.py:1493-1660``, ``sharding/rw_sequence_sharding.py:44-160``).
Here the input distribution of ``FusedSparseEngine`` additionally tags every id with a *return address*
``(requesting rank << 32) | position of the id in the requester's KJT``, and

    lookup     every owner stores the row of each received id straight into row ``position`` of the requester's output
               buffer, at the shard's column offset (column-wise shards of one table fill disjoint columns of the same row;
               row-wise shards fill disjoint rows); no output all-to-all, no un-bucketize permutation
    finalize   rows ``[0, n)`` of the buffer are copied out (cast, NaN-poisoned after a failed wait) as ``[n, D]``
    backward   the requester copies its ``[n, D]`` output gradient into a peer-readable buffer; every owner's TBE backward
               pulls the gradient row of each id through the same return address while it applies the fused optimizer

Rows come out in the order of the requester's own KJT values, so cutting them into per-feature ``JaggedTensor`` s needs only
the KJT's own lengths.  Table-wise, column-wise and row-wise shards are all (rows x columns) blocks and share the code.
"""
from __future__ import annotations

from typing import Any, Optional, Sequence

import torch

from torchrec_b200.distributed.fused_sparse_engine import (
    SLOT_FIN,
    SLOT_GRAD,
    SLOT_OUT,
    DistHandle,
    FusedSparseEngine,
    _Buffers,
    dist_slack,
)
from torchrec_b200.distributed.peer_memory import _PeerBase


class FusedSequenceEngine(FusedSparseEngine):
    """See the module docstring.  Built by ``ShardedEmbeddingCollection``."""

    sequence = True

    def __init__(self, peer: _PeerBase, table_configs: Sequence[Any], shardings: Sequence[Any], lookups: Sequence[Any],
                 out_dtype: torch.dtype, stage_dtype: torch.dtype, grad_dtype: torch.dtype) -> None:
        dims = {int(c.embedding_dim) for c in table_configs}
        assert len(dims) == 1 and next(iter(dims)) % 4 == 0, "one embedding dim (a multiple of 4) for all tables"
        super().__init__(peer, table_configs, shardings, lookups, out_dtype, stage_dtype, grad_dtype)
        assert not any(m.weighted for m in self.modules)
        self.solo = self.W == 1  # one rank: the lookup writes the result tensor itself and reads the gradient tensor itself

    # ------------------------------------------------------------------------------------------------------------------
    def _alloc_sequence_buffers(self, b: _Buffers) -> None:
        if self.W == 1:
            b.out_rows = 0
            return
        b.out_rows = max(1024, (int(b.max_values * dist_slack()) + 1023) // 1024 * 1024)
        b.seq_out, b.seq_out_ptrs = self.peer.alloc_shared((b.out_rows, self.total_D), self.stage_dtype)
        b.seq_grad, b.seq_grad_ptrs = self.peer.alloc_shared((b.out_rows, self.total_D), self.grad_dtype)

    def _rows_of(self, h: DistHandle, b: _Buffers) -> int:
        n = int(h.values.numel())
        if not self.solo and n > b.out_rows:
            raise RuntimeError(f"this batch holds {n} ids but the sequence output buffer was sized for {b.out_rows}; raise TRB200_DIST_SLACK")
        return n

    # ------------------------------------------------------------------------------------------------------------------
    def phase_push(self, h: DistHandle, build_plans: bool) -> None:
        b = self._bufs[h.B]
        r = b.recv[h.parity]
        Bg = self.W * h.B
        n = self._rows_of(h, b)
        n_jobs = self.dest_job_start[self.rank + 1] - self.dest_job_start[self.rank]
        roff = torch.ops.trb200.kjt_dist_recv_offsets(r.len, n_jobs * Bg, self.ids_dtype == torch.int64, self.flags.ptrs, self.rank,
                                                     self.flags.epochs, self.peer.wait_cycles, self.peer.err)
        h.recv_offsets = roff
        if self.solo:
            h.out = torch.zeros((n, self.total_D), dtype=self.out_dtype, device=self.device)
            dst_ptrs, rows, dst_dtype = [h.out.data_ptr()], n, self.out_dtype
        else:
            # every rank has copied the previous step's rows out before they are overwritten
            self.flags.wait(SLOT_FIN)
            dst_ptrs, rows, dst_dtype = b.seq_out_ptrs, b.out_rows, self.stage_dtype
        h.plans = []
        for m in self.modules:
            off = roff[m.j0 * Bg: m.j1 * Bg + 1]
            m.tbe.seq_forward_push(r.val, off, r.ret, Bg, dst_ptrs, rows, self.total_D, m.bwd_cols, dst_dtype)
            h.plans.append(m.tbe.build_plan_ahead(r.val, off, None, Bg, padded=True) if build_plans else None)
        if not self.solo:
            self.flags.signal(SLOT_OUT)

    def phase_finalize(self, h: DistHandle) -> torch.Tensor:
        b = self._bufs[h.B]
        if self.solo:
            out, h.out = h.out, None
            return out
        self.flags.wait(SLOT_OUT)
        out = torch.ops.trb200.seq_finalize(b.seq_out, int(h.values.numel()), self.out_dtype, self.peer.err)
        self.flags.signal(SLOT_FIN)
        return out

    def phase_publish(self, h: DistHandle, grad: torch.Tensor, scale: float = 1.0) -> None:
        b = self._bufs[h.B]
        h.scale = scale
        if self.solo:
            h.grad = grad.contiguous()
            return
        b.seq_grad[: grad.shape[0]].copy_(grad)
        self.flags.signal(SLOT_GRAD)

    def phase_pull(self, h: DistHandle) -> None:
        b = self._bufs[h.B]
        r = b.recv[h.parity]
        Bg = self.W * h.B
        if self.solo:
            grad, ptrs = h.grad, [h.grad.data_ptr()]
            h.grad = None
        else:
            self.flags.wait(SLOT_GRAD)
            grad, ptrs = b.seq_grad, b.seq_grad_ptrs
        for m, plan in zip(self.modules, h.plans):
            off = h.recv_offsets[m.j0 * Bg: m.j1 * Bg + 1]
            m.tbe.seq_backward_pull(grad, ptrs, r.ret, r.val, off, Bg, m.bwd_cols, float(getattr(h, "scale", 1.0)), plan)
        if not torch.cuda.is_current_stream_capturing():
            ev = torch.cuda.Event()
            ev.record()
            self._consumed[h.parity] = ev
