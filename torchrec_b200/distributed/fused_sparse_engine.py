"""Fused sparse engine: one sharded ``EmbeddingBagCollection`` step as a handful of kernels over peer-mapped memory.

For the ranks of one node the engine replaces the per-sharding-type chain of the classic path (split-size all-to-all +
host read, one all-to-all per KJT tensor, permute, lookup, pooled all-to-all / reduce-scatter, column permute) by

    input_dist   ``kjt_dist_send`` x2: count + publish sizes, then write lengths / ids / weights straight into every
                 destination's receive buffer (row-split tables are bucketized on the fly); sizes never reach the host
    lookup       the TBE forward of every local table group stores each pooled bag into the *owner's* staging row
                 (whole-shard tables at their final output column, row-split tables into a per-source partial slot)
    finalize     one kernel per rank sums the partial slots in a fixed order, applies mean divisors, casts, and
                 writes a fresh ``[B_local, sum(D)]`` output in the unsharded module's column order
    backward     ``grad_publish`` pushes every column block of the output gradient into the local gradient slab of the
                 rank(s) that own the table; every owner's TBE backward then segment-reduces rows of its own slab while
                 it applies the fused optimizer (no gradient all-to-all call, no ``[ids, D]`` tensor)

All sharding types whose shards are (rows x columns) blocks of a table are covered by one mechanism: table-wise,
column-wise, table-column-wise, row-wise, table-row-wise and grid shards are just different block layouts.  Data-
parallel tables, feature processors, variable batch per feature and non-fused optimizers stay on the classic path.

Receive buffers have a fixed capacity (measured on the first batch times ``TRB200_DIST_SLACK``, default 1.25), ids past
the real count are padding that the backward skips through a device-side count, and flag epochs are counted on the
device; so a step issues no host synchronisation and can be captured in a CUDA graph.

Stream contract: ``input_dist`` may run on a side stream ahead of time (two alternating receive buffers); ``lookup`` and
its backward run on the compute stream, and a step's backward is enqueued before the next step's ``lookup``.

Reference counterparts: ``torchrec/distributed/embeddingbag.py:1463-1640`` (the three stages),
``torchrec/distributed/dist_data.py:220-442`` and ``:897-1490`` (the collectives this replaces).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from torchrec_b200.distributed.peer_memory import FlagSet, _PeerBase
from torchrec_b200.modules.embedding_configs import PoolingMode, PoolingType
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

SLOT_SIZES, SLOT_DATA, SLOT_OUT, SLOT_FIN, SLOT_GRAD = 0, 1, 2, 3, 4
_NSLOTS = 8
_CHUNK = 256


def dist_slack() -> float:
    return float(os.environ.get("TRB200_DIST_SLACK", "1.25"))


@dataclass
class _Job:
    dest: int
    local: int          # position among the destination's jobs
    feature: str
    table: str
    row_lo: int
    row_hi: int
    col_off: int
    cols: int
    whole: bool
    out_col: int        # first output column of (table, feature) in the unsharded module's output
    mean_after: bool    # mean pooling applied at finalize (the kernel pools with SUM)
    module: Tuple[int, int]  # (sharding index, group index) at the destination
    slot: int = -1
    shard_index: int = -1    # index into grp_jobs for row-split jobs


@dataclass
class _ModuleRange:
    tbe: Any
    weighted: bool
    j0: int
    j1: int
    fwd_cols: List[int] = field(default_factory=list)   # staging column of every feature (forward)
    bwd_cols: List[int] = field(default_factory=list)   # column in the module's output (= in its gradient)
    slab_cols: List[int] = field(default_factory=list)  # column in this rank's gradient slab


class DistHandle:
    """Result of ``input_dist``: which receive buffers hold the batch and what the later phases need from the KJT."""

    def __init__(self, parity: int, B: int, offsets: torch.Tensor, values: torch.Tensor, weights: Optional[torch.Tensor], feat_pos: torch.Tensor) -> None:
        self.parity = parity
        self.B = B
        self.offsets = offsets
        self.values = values
        self.weights = weights
        self.feat_pos = feat_pos
        self.recv_offsets: Optional[torch.Tensor] = None
        self.plans: List[Any] = []
        self.out: Optional[torch.Tensor] = None   # one-rank shortcut: the lookups write the output directly
        self.grad: Optional[torch.Tensor] = None  # ... and read the output gradient directly

    def record_stream(self, stream: torch.Stream) -> None:
        for t in (self.offsets, self.values, self.weights, self.feat_pos):
            if t is not None and t.is_cuda:
                t.record_stream(stream)


class _Buffers:
    pass


class FusedSparseEngine:
    """See the module docstring.  Built by ``ShardedEmbeddingBagCollection`` through :meth:`build`."""

    sequence = False  # the unpooled variant (``FusedSequenceEngine``) lays its output out per id, not per bag

    def __init__(self, peer: _PeerBase, table_configs: Sequence[Any], shardings: Sequence[Any], lookups: Sequence[Any],
                 out_dtype: torch.dtype, stage_dtype: torch.dtype, grad_dtype: torch.dtype) -> None:
        self.peer = peer
        self.W, self.rank, self.device = peer.world, peer.rank, peer.device
        self.out_dtype, self.stage_dtype, self.grad_dtype = out_dtype, stage_dtype, grad_dtype
        self._build_jobs(table_configs, shardings, lookups)
        self.flags: FlagSet = peer.new_flags(_NSLOTS)
        self._bufs: Dict[int, _Buffers] = {}
        self._feat_pos_cache: Dict[Tuple[str, ...], torch.Tensor] = {}
        self._calls = 0
        self._consumed: List[Optional[torch.cuda.Event]] = [None, None]
        self._anchor = torch.zeros(1, requires_grad=True)
        self.ids_dtype: Optional[torch.dtype] = None
        self.weighted = any(m.weighted for m in self.modules)
        self.recv_counts: List[int] = []
        # optional per-phase device timing (benchmarks): phase -> list of (start event, end event)
        self.timing: Optional[Dict[str, List[Tuple[torch.cuda.Event, torch.cuda.Event]]]] = None

    def _timed(self, phase: str):
        """Context manager that brackets a phase with CUDA events when ``timing`` is on."""
        import contextlib

        if self.timing is None or torch.cuda.is_current_stream_capturing():
            return contextlib.nullcontext()
        engine = self

        class _T:
            def __enter__(self_inner):
                self_inner.e0 = torch.cuda.Event(enable_timing=True)
                self_inner.e0.record()

            def __exit__(self_inner, *exc):
                e1 = torch.cuda.Event(enable_timing=True)
                e1.record()
                engine.timing.setdefault(phase, []).append((self_inner.e0, e1))

        return _T()

    def timing_summary(self) -> Dict[str, float]:
        """Mean device milliseconds per phase since ``timing`` was switched on (synchronises)."""
        torch.cuda.synchronize(self.device)
        return {k: sum(a.elapsed_time(b) for a, b in v) / max(len(v), 1) for k, v in (self.timing or {}).items()}

    # ------------------------------------------------------------------------------------------------------------------
    # static layout
    # ------------------------------------------------------------------------------------------------------------------
    def _build_jobs(self, table_configs, shardings, lookups) -> None:
        W = self.W
        # output columns in the unsharded module's order; a feature shared by two tables appears once per table
        out_col: Dict[Tuple[str, str], int] = {}
        pooling_of: Dict[str, Any] = {}
        rows_of: Dict[str, int] = {}
        acc = 0
        for cfg in table_configs:
            pooling_of[cfg.name] = getattr(cfg, "pooling", None)
            rows_of[cfg.name] = cfg.num_embeddings
            for f in (cfg.feature_names or [cfg.name]):
                if self.sequence:  # one output row per id: every table starts at column 0 of it
                    assert not any(k[1] == f for k in out_col), f"feature {f} feeds two tables"
                    out_col[(cfg.name, f)] = 0
                    acc = max(acc, cfg.embedding_dim)
                else:
                    out_col[(cfg.name, f)] = acc
                    acc += cfg.embedding_dim
        self.total_D = acc
        jobs: List[_Job] = []
        self.dest_job_start = [0]
        for d in range(W):
            j = 0
            for si, sh in enumerate(shardings):
                for gi, group in enumerate(sh._grouped_embedding_configs_per_rank[d]):
                    pooling_sum = None
                    for t in group.embedding_tables:
                        ro, co = t.local_metadata.shard_offsets
                        rs, cs = t.local_metadata.shard_sizes
                        total_rows = int(t.global_metadata.size[0]) if t.global_metadata is not None else rows_of[t.name]
                        for f in t.feature_names:
                            jobs.append(_Job(dest=d, local=j, feature=f, table=t.name, row_lo=int(ro), row_hi=int(ro + rs), col_off=int(co),
                                             cols=int(cs), whole=(int(rs) == total_rows and int(ro) == 0), out_col=out_col[(t.name, f)],
                                             mean_after=False, module=(si, gi)))
                            j += 1
            self.dest_job_start.append(self.dest_job_start[-1] + j)
        # the kernels move four elements at a time: every column block must start and end on a multiple of 4
        assert all(jb.cols % 4 == 0 and jb.col_off % 4 == 0 and jb.out_col % 4 == 0 for jb in jobs), "embedding dims and column shards must be multiples of 4"
        self.jobs = jobs
        self.G = len(jobs)
        self.J_max = max((self.dest_job_start[d + 1] - self.dest_job_start[d] for d in range(W)), default=0)
        # feature slots
        slots: Dict[str, int] = {}
        for jb in jobs:
            jb.slot = slots.setdefault(jb.feature, len(slots))
        self.slot_names = list(slots.keys())
        # local modules, in the order of this rank's jobs
        self.modules: List[_ModuleRange] = []
        g0 = self.dest_job_start[self.rank]
        j = 0
        for si, (sh, lk) in enumerate(zip(shardings, lookups)):
            groups = sh._grouped_embedding_configs_per_rank[self.rank]
            embs = list(lk.emb_modules)
            assert len(groups) == len(embs), "lookup groups do not match the sharding's groups"
            for gi, (group, emb) in enumerate(zip(groups, embs)):
                n = group.num_features()
                self.modules.append(_ModuleRange(tbe=emb.emb_module, weighted=bool(group.is_weighted), j0=j, j1=j + n))
                j += n
        assert j == self.dest_job_start[self.rank + 1] - g0
        # mean-after-reduction: the table pools with MEAN but its kernel was built to SUM (row-split shardings)
        for d in range(W):
            for si, sh in enumerate(shardings):
                for gi, group in enumerate(sh._grouped_embedding_configs_per_rank[d]):
                    from torchrec_b200.modules.embedding_configs import pooling_type_to_pooling_mode

                    kernel_mode = pooling_type_to_pooling_mode(group.pooling, getattr(sh, "sharding_type", None))
                    if group.pooling.value == PoolingType.MEAN.value and kernel_mode == PoolingMode.SUM:
                        for jb in jobs:
                            if jb.dest == d and jb.module == (si, gi):
                                jb.mean_after = True
        # row-split features: groups of jobs that share (table, feature, column block)
        groups_by_key: Dict[Tuple[str, str, int], List[int]] = {}
        for g, jb in enumerate(jobs):
            if not jb.whole:
                groups_by_key.setdefault((jb.table, jb.feature, jb.col_off), []).append(g)
        self.grp: List[Tuple[int, int, int]] = []
        self.grp_jobs: List[int] = []
        self.part_col: Dict[Tuple[str, str, int], int] = {}
        P = 0
        for key, gs in groups_by_key.items():
            gs.sort(key=lambda g: jobs[g].row_lo)
            assert len(gs) <= 16, "at most 16 row ranges per table"
            assert jobs[gs[0]].row_lo == 0 and all(jobs[a].row_hi == jobs[b].row_lo for a, b in zip(gs, gs[1:])), f"row shards of {key} are not contiguous"
            assert len({jobs[g].dest for g in gs}) == len(gs), f"two row shards of {key} on one rank"
            self.grp.append((jobs[gs[0]].slot, len(self.grp_jobs), len(gs)))
            for k, g in enumerate(gs):
                jobs[g].shard_index = len(self.grp_jobs)
                self.grp_jobs.append(g)
            self.part_col[key] = P
            P += jobs[gs[0]].cols
        self.P = P
        self.Q = len(self.grp)
        self.whole_jobs = [g for g, jb in enumerate(jobs) if jb.whole]
        self.stage_cols = self.total_D + W * P
        # per local module: staging column of every feature in forward, gradient column in backward
        for m in self.modules:
            for jb in jobs[g0 + m.j0: g0 + m.j1]:
                final = jb.out_col + jb.col_off
                m.bwd_cols.append(final)
                m.fwd_cols.append(final if jb.whole else self.total_D + self.rank * P + self.part_col[(jb.table, jb.feature, jb.col_off)])
        # finalize / publish segments: (out col, width, staging col, parts, part stride, mean feature slot)
        segs: List[List[int]] = []
        seen = set()
        for jb in jobs:
            key = (jb.table, jb.feature, jb.col_off)
            if key in seen:
                continue
            seen.add(key)
            final = jb.out_col + jb.col_off
            mean_slot = jb.slot if jb.mean_after else -1
            if jb.whole:
                segs.append([final, jb.cols, final, 1, 0, mean_slot])
            else:
                segs.append([final, jb.cols, self.total_D + self.part_col[key], W, P, mean_slot])
        # gradient slabs: on its owner, job g reads columns [slab_col, slab_col + cols) of row (source rank * B + b)
        gsegs: List[List[int]] = []
        self.slab_cols = 4
        slab_col_of: Dict[int, int] = {}
        for d in range(W):
            acc = 0
            for g in range(self.dest_job_start[d], self.dest_job_start[d + 1]):
                jb = jobs[g]
                slab_col_of[g] = acc
                gsegs.append([jb.out_col + jb.col_off, jb.cols, d, acc, jb.slot if jb.mean_after else -1])
                acc += jb.cols
            self.slab_cols = max(self.slab_cols, acc)
        for m in self.modules:
            m.slab_cols = [slab_col_of[g0 + j] for j in range(m.j0, m.j1)]
        self.has_mean_after = any(jb.mean_after for jb in jobs)
        # one rank and nothing to fix up afterwards: lookups write the output and read the gradient directly
        self.direct = W == 1 and not self.has_mean_after and not self.sequence
        covered = sum(s[1] for s in segs)
        assert self.sequence or covered == self.total_D, f"shards cover {covered} of {self.total_D} output columns"
        dev = self.device
        i32 = dict(dtype=torch.int32, device=dev)
        self.t_seg = torch.tensor(segs, **i32).reshape(-1, 6)
        self.t_gseg = torch.tensor(gsegs, **i32).reshape(-1, 5)
        self.t_jobs = torch.tensor([[jb.dest, jb.local, jb.slot, 0 if jb.whole else 1, max(jb.shard_index, 0)] for jb in jobs], **i32).reshape(-1, 5)
        self.t_dest_job_start = torch.tensor(self.dest_job_start, **i32)
        self.t_grp = torch.tensor(self.grp, **i32).reshape(-1, 3)
        self.t_grp_jobs = torch.tensor(self.grp_jobs, **i32)
        self.t_whole = torch.tensor(self.whole_jobs, **i32)
        self.t_row_lo = torch.tensor([jb.row_lo for jb in jobs], dtype=torch.int64, device=dev)
        self.t_row_hi = torch.tensor([jb.row_hi for jb in jobs], dtype=torch.int64, device=dev)

    # ------------------------------------------------------------------------------------------------------------------
    # buffers
    # ------------------------------------------------------------------------------------------------------------------
    def accepts(self, kjt: KeyedJaggedTensor) -> bool:
        if kjt.variable_stride_per_key() or kjt.stride() <= 0 or not kjt.values().is_cuda:
            return False
        have = set(kjt.keys())
        return all(n in have for n in self.slot_names)

    def _feat_pos(self, kjt: KeyedJaggedTensor) -> torch.Tensor:
        key = tuple(kjt.keys())
        t = self._feat_pos_cache.get(key)
        if t is None:
            index = {k: i for i, k in enumerate(key)}
            t = torch.tensor([index[n] for n in self.slot_names], dtype=torch.int32, device=self.device)
            self._feat_pos_cache[key] = t
        return t

    def _topo(self, feat_pos: torch.Tensor) -> List[torch.Tensor]:
        return [self.t_jobs, self.t_dest_job_start, self.t_grp, self.t_grp_jobs, self.t_whole, feat_pos]

    def _weights_of(self, kjt: KeyedJaggedTensor) -> Optional[torch.Tensor]:
        if not self.weighted:
            return None
        w = kjt.weights_or_none()
        if w is None or not torch.is_floating_point(w):
            return None
        return w if w.dtype == torch.float32 else w.float()

    def _ids_of(self, kjt: KeyedJaggedTensor) -> torch.Tensor:
        v = kjt.values()
        if self.ids_dtype is None:
            self.ids_dtype = v.dtype if v.dtype in (torch.int32, torch.int64) else torch.int64
        return v if v.dtype == self.ids_dtype else v.to(self.ids_dtype)

    def prepare(self, kjt: KeyedJaggedTensor) -> None:
        """First half of sizing the buffers for per-rank batch size ``B`` (collective): allocates the small tables and
        counts this batch.  ``prepare_finish`` reads the counts and allocates the receive buffers."""
        B = kjt.stride()
        nshards = max(len(self.grp_jobs), 1)
        nchunks = (B + _CHUNK - 1) // _CHUNK
        b = _Buffers()
        b.B = B
        b.sizes, b.sizes_ptrs = self.peer.alloc_shared((2 * self.W * (self.G + 2),), torch.int32)
        b.send_len = torch.zeros(nshards * B, dtype=torch.int32, device=self.device)
        b.chunk_sum = torch.zeros(nshards * nchunks, dtype=torch.int32, device=self.device)
        b.counters = torch.zeros(2, dtype=torch.int32, device=self.device)
        b.cap = 0
        b.recv = []
        self._bufs[B] = b
        self._pending = (b, kjt)
        self._send(b, kjt, 0, probe=True)

    def prepare_finish(self) -> None:
        b, kjt = self._pending
        self._pending = None
        torch.cuda.synchronize(self.device)
        pg = getattr(self.peer, "pg", None)
        if pg is not None:
            import torch.distributed as dist

            dist.barrier(group=pg)
        epoch = int(self.flags.epochs[SLOT_SIZES].item())
        S = b.sizes.view(2, self.W, self.G + 2)[epoch & 1].cpu()
        recv = [int(S[:, self.dest_job_start[d]: self.dest_job_start[d + 1]].sum()) for d in range(self.W)]
        self.recv_counts = recv  # ids every rank's lookup receives for the batch that sized the buffers
        b.max_values = int(S[:, self.G + 1].max())  # largest KJT (ids of all its features) over the ranks
        b.cap = max(1024, (int(max(recv) * dist_slack()) + 1023) // 1024 * 1024)
        ids_dtype = self.ids_dtype or torch.int64
        n_len = max(self.J_max * self.W * b.B, 1)
        for _ in range(2):
            r = _Buffers()
            r.len, r.len_ptrs = self.peer.alloc_shared((n_len,), torch.int32)
            r.val, r.val_ptrs = self.peer.alloc_shared((b.cap,), ids_dtype)
            if self.weighted:
                r.w, r.w_ptrs = self.peer.alloc_shared((b.cap,), torch.float32)
            else:
                r.w, r.w_ptrs = None, []
            if self.sequence:
                r.ret, r.ret_ptrs = self.peer.alloc_shared((b.cap,), torch.int64)
            else:
                r.ret, r.ret_ptrs = None, []
            b.recv.append(r)
        if self.sequence:
            self._alloc_sequence_buffers(b)
        elif not self.direct:
            b.staging, b.staging_ptrs = self.peer.alloc_shared((b.B, self.stage_cols), self.stage_dtype)
            b.gslab, b.gslab_ptrs = self.peer.alloc_shared((self.W * b.B, self.slab_cols), self.grad_dtype)
        if pg is not None:
            import torch.distributed as dist

            dist.barrier(group=pg)

    def _send(self, b: _Buffers, kjt: KeyedJaggedTensor, phase: int, probe: bool = False, handle: Optional[DistHandle] = None) -> None:
        if handle is not None:
            offsets, values, weights, feat_pos = handle.offsets, handle.values, handle.weights, handle.feat_pos
            r = b.recv[handle.parity]
        else:
            offsets, values, weights, feat_pos = kjt.offsets(), self._ids_of(kjt), self._weights_of(kjt), self._feat_pos(kjt)
            r = None
        if probe:
            len_ptrs = val_ptrs = b.sizes_ptrs  # phase 0 touches neither
            w_ptrs = b.sizes_ptrs if weights is not None else []
            ret_ptrs: List[int] = []
            cap = 0
        else:
            len_ptrs, val_ptrs, w_ptrs, cap = r.len_ptrs, r.val_ptrs, (r.w_ptrs if weights is not None else []), b.cap
            ret_ptrs = r.ret_ptrs
        torch.ops.trb200.kjt_dist_send(
            phase, self.rank, b.B, self._topo(feat_pos), [self.t_row_lo, self.t_row_hi], [b.send_len, b.chunk_sum, b.counters, self.flags.epochs],
            values, offsets, weights, self.flags.ptrs, b.sizes_ptrs, len_ptrs, val_ptrs, w_ptrs, ret_ptrs, cap, self.peer.wait_cycles, self.peer.err,
        )

    # ------------------------------------------------------------------------------------------------------------------
    # phases (a real rank runs them back to back; an emulation runs each phase for all virtual ranks before the next)
    # ------------------------------------------------------------------------------------------------------------------
    def new_handle(self, kjt: KeyedJaggedTensor) -> DistHandle:
        B = kjt.stride()
        if B not in self._bufs:
            raise RuntimeError("call prepare()/prepare_finish() (or input_dist) first for this batch size")
        parity = self._calls & 1
        self._calls += 1
        h = DistHandle(parity, B, kjt.offsets(), self._ids_of(kjt), self._weights_of(kjt), self._feat_pos(kjt))
        capturing = torch.cuda.is_current_stream_capturing()
        ev = self._consumed[parity]
        if ev is not None and not capturing:
            torch.cuda.current_stream().wait_event(ev)
        return h

    def phase_send(self, h: DistHandle, phase: int) -> None:
        self._send(self._bufs[h.B], None, phase, handle=h)

    def input_dist(self, kjt: KeyedJaggedTensor) -> DistHandle:
        with torch.no_grad():
            if kjt.stride() not in self._bufs:
                self.prepare(kjt)
                self.prepare_finish()
            h = self.new_handle(kjt)
            with self._timed("input_dist"):
                self.phase_send(h, 0)
                self.phase_send(h, 1)
        return h

    def phase_push(self, h: DistHandle, build_plans: bool) -> None:
        b = self._bufs[h.B]
        r = b.recv[h.parity]
        Bg = self.W * h.B
        n_jobs = self.dest_job_start[self.rank + 1] - self.dest_job_start[self.rank]
        roff = torch.ops.trb200.kjt_dist_recv_offsets(r.len, n_jobs * Bg, self.ids_dtype == torch.int64, self.flags.ptrs, self.rank,
                                                     self.flags.epochs, self.peer.wait_cycles, self.peer.err)
        h.recv_offsets = roff
        if self.direct:
            h.out = torch.empty((h.B, self.total_D), dtype=self.out_dtype, device=self.device)
            dst_ptrs, dst_stride, dst_dtype = [h.out.data_ptr()], self.total_D, self.out_dtype
        else:
            # every rank has finished reading the staging rows of the previous step before they are overwritten
            self.flags.wait(SLOT_FIN)
            dst_ptrs, dst_stride, dst_dtype = b.staging_ptrs, self.stage_cols, self.stage_dtype
        h.plans = []
        for m in self.modules:
            off = roff[m.j0 * Bg: m.j1 * Bg + 1]
            psw = r.w if (m.weighted and h.weights is not None) else None
            m.tbe.forward_push(r.val, off, psw, Bg, h.B, dst_ptrs, dst_stride, m.bwd_cols if self.direct else m.fwd_cols, dst_dtype)
            h.plans.append(m.tbe.build_plan_ahead(r.val, off, psw, Bg, padded=True) if build_plans else None)
        if not self.direct:
            self.flags.signal(SLOT_OUT)

    def phase_finalize(self, h: DistHandle) -> torch.Tensor:
        b = self._bufs[h.B]
        if self.direct:
            out, h.out = h.out, None
            return out
        self.flags.wait(SLOT_OUT)
        out = torch.ops.trb200.pooled_finalize(b.staging, self.stage_cols, self.t_seg, h.B, self.total_D, self.out_dtype, h.offsets, h.feat_pos,
                                               self.peer.err)
        self.flags.signal(SLOT_FIN)
        return out

    def phase_publish(self, h: DistHandle, grad: torch.Tensor, scale: float = 1.0) -> None:
        b = self._bufs[h.B]
        if grad.dim() != 2 or grad.stride(1) != 1 or grad.data_ptr() % 16 != 0 or (grad.stride(0) * grad.element_size()) % 16 != 0:
            grad = grad.contiguous()
        if self.direct:
            h.grad = grad
            return
        torch.ops.trb200.grad_publish(grad, b.gslab_ptrs, self.grad_dtype, self.slab_cols, self.rank, self.t_gseg, h.offsets, h.feat_pos, scale)
        self.flags.signal(SLOT_GRAD)

    def phase_pull(self, h: DistHandle) -> None:
        b = self._bufs[h.B]
        r = b.recv[h.parity]
        Bg = self.W * h.B
        if self.direct:
            grad = h.grad
            h.grad = None
        else:
            self.flags.wait(SLOT_GRAD)
            grad = b.gslab
        for m, plan in zip(self.modules, h.plans):
            off = h.recv_offsets[m.j0 * Bg: m.j1 * Bg + 1]
            psw = r.w if (m.weighted and h.weights is not None) else None
            m.tbe.backward_local(grad, r.val, off, psw, Bg, m.bwd_cols if self.direct else m.slab_cols, plan, padded=True)
        if not torch.cuda.is_current_stream_capturing():
            ev = torch.cuda.Event()
            ev.record()
            self._consumed[h.parity] = ev

    # ------------------------------------------------------------------------------------------------------------------
    # autograd entry
    # ------------------------------------------------------------------------------------------------------------------
    def lookup(self, h: DistHandle) -> torch.Tensor:
        """Pooled output ``[B_local, sum(D)]`` of the batch behind ``h`` in the unsharded module's column order."""
        if torch.is_grad_enabled():
            return _EngineLookup.apply(self._anchor, self, h)
        self.phase_push(h, build_plans=False)
        out = self.phase_finalize(h)
        if not torch.cuda.is_current_stream_capturing():
            ev = torch.cuda.Event()
            ev.record()
            self._consumed[h.parity] = ev
        return out

    def forward(self, kjt: KeyedJaggedTensor) -> torch.Tensor:
        return self.lookup(self.input_dist(kjt))


class _EngineLookup(torch.autograd.Function):
    @staticmethod
    def forward(ctx, anchor, engine: FusedSparseEngine, h: DistHandle):
        with engine._timed("lookup_push"):
            engine.phase_push(h, build_plans=True)
        with engine._timed("finalize"):
            out = engine.phase_finalize(h)
        ctx.engine, ctx.h = engine, h
        return out

    @staticmethod
    def backward(ctx, grad):
        from torchrec_b200.distributed import comm_ops

        engine, h = ctx.engine, ctx.h
        scale = 1.0 / engine.W if comm_ops.get_gradient_division() else 1.0
        with engine._timed("grad_publish"):
            engine.phase_publish(h, grad, scale)
        with engine._timed("backward_update"):
            engine.phase_pull(h)
        ctx.h = None
        return None, None, None
