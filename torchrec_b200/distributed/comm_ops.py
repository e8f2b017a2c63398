"""Autograd-aware collectives for embedding outputs (NCCL / gloo path).

Every collective is a pair of autograd functions: ``*_Req`` launches the forward collective
asynchronously and returns a dummy tensor; ``*_Wait`` waits and post-processes.  In backward the
roles swap -- ``Wait.backward`` launches the gradient collective and ``Req.backward`` waits for it
-- so the gradient communication overlaps with whatever autograd runs in between.  Optional codecs
cast/quantise the payload around the collective with independent forward/backward precision.

Same protocol and shapes as ``torchrec/distributed/comm_ops.py`` (pooled all-to-all ``:337,1134-1376``,
sequence all-to-all ``:1597-1802``, reduce-scatter / all-gather ``:803-1020,2038-2351``).  These are
the *baseline* collectives; the fused sm_100a paths in ``torchrec_b200.parallel`` replace them on
NVLink-connected GPUs.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor
from torch.autograd import Function
from torch.autograd.profiler import record_function

from torchrec_b200.distributed.types import Awaitable, NoWait, QuantizedCommCodecs
from torchrec_b200.ops import sparse_ops as sops

GRADIENT_DIVISION: bool = True
USE_SYNC_COLLECTIVES: bool = False


def set_gradient_division(val: bool) -> None:
    """Divide embedding gradients by the world size in the backward collectives (matches DDP averaging)."""
    global GRADIENT_DIVISION
    GRADIENT_DIVISION = val


def get_gradient_division() -> bool:
    return GRADIENT_DIVISION


def set_use_sync_collectives(val: bool) -> None:
    global USE_SYNC_COLLECTIVES
    USE_SYNC_COLLECTIVES = val


def get_use_sync_collectives() -> bool:
    return USE_SYNC_COLLECTIVES


def _backend_is_gloo(pg: Optional[dist.ProcessGroup]) -> bool:
    try:
        return "gloo" in str(dist.get_backend(pg))
    except Exception:
        return False


# ---- raw collectives with a gloo fallback where gloo lacks the primitive --------------------------
def _all_to_all_single(out: Tensor, inp: Tensor, out_splits, in_splits, pg, async_op: bool):
    return dist.all_to_all_single(out, inp, output_split_sizes=out_splits, input_split_sizes=in_splits, group=pg, async_op=async_op)


class _DoneWork:
    def wait(self) -> None:
        return None


def _reduce_scatter_tensor(out: Tensor, inp: Tensor, pg, async_op: bool):
    """``inp [W*n] -> out [n]`` summed over ranks."""
    if _backend_is_gloo(pg) or not inp.is_cuda:
        W = dist.get_world_size(pg)
        recv = torch.empty_like(inp)
        dist.all_to_all_single(recv, inp.contiguous(), group=pg)
        out.copy_(recv.view(W, -1).sum(0).view_as(out))
        return _DoneWork()
    return dist.reduce_scatter_tensor(out, inp, group=pg, async_op=async_op)


def _reduce_scatter_v(out: Tensor, inp: Tensor, in_splits_rows: List[int], pg, async_op: bool):
    """Uneven reduce-scatter over dim 0: rank r receives the sum of everyone's rows ``[off_r, off_r+n_r)``."""
    W = dist.get_world_size(pg)
    rank = dist.get_rank(pg)
    row = inp[0].numel() if inp.dim() > 1 else 1
    recv = torch.empty((W * in_splits_rows[rank],) + tuple(inp.shape[1:]), dtype=inp.dtype, device=inp.device)
    dist.all_to_all_single(
        recv, inp.contiguous(), output_split_sizes=[in_splits_rows[rank]] * W, input_split_sizes=list(in_splits_rows), group=pg,
    )
    del row
    out.copy_(recv.view((W, in_splits_rows[rank]) + tuple(inp.shape[1:])).sum(0))
    return _DoneWork()


def _all_gather_into_tensor(out: Tensor, inp: Tensor, pg, async_op: bool):
    return dist.all_gather_into_tensor(out, inp.contiguous(), group=pg, async_op=async_op)


# ---- request plumbing ----------------------------------------------------------------------------
class Request(Awaitable[Tensor]):
    """Handle of one in-flight collective; ``wait()`` runs the matching ``*_Wait`` function."""

    def __init__(self, pg: dist.ProcessGroup, device: torch.device) -> None:
        super().__init__()
        self.pg = pg
        self.req = None
        self.tensor: Optional[Tensor] = None
        self.info: Any = None
        self.qcomm_ctx = None
        self.wait_function = None
        self.dummy_tensor: Tensor = torch.empty(1, requires_grad=True, device=device)

    def _wait_impl(self) -> Tensor:
        ret = self.wait_function.apply(self.pg, self, self.dummy_tensor)
        self.req = None
        self.tensor = None
        return ret


@dataclass
class All2AllPooledInfo:
    batch_size_per_rank: List[int]
    dim_sum_per_rank: List[int]
    dim_sum_per_rank_tensor: Optional[Tensor]
    cumsum_dim_sum_per_rank_tensor: Optional[Tensor]
    codecs: Optional[QuantizedCommCodecs] = None


@dataclass
class VariableBatchAll2AllPooledInfo:
    batch_size_per_rank_per_feature: List[List[int]]
    batch_size_per_feature_pre_a2a: List[int]
    emb_dim_per_rank_per_feature: List[List[int]]
    codecs: Optional[QuantizedCommCodecs] = None
    input_splits: Optional[List[int]] = None
    output_splits: Optional[List[int]] = None


@dataclass
class All2AllSequenceInfo:
    embedding_dim: int
    lengths_after_sparse_data_all2all: Tensor
    forward_recat_tensor: Optional[Tensor]
    backward_recat_tensor: Tensor
    input_splits: List[int]
    output_splits: List[int]
    variable_batch_size: bool = False
    codecs: Optional[QuantizedCommCodecs] = None
    permuted_lengths_after_sparse_data_all2all: Optional[Tensor] = None


@dataclass
class All2AllVInfo:
    dims_sum_per_rank: List[int]
    B_global: int
    B_local: int
    B_local_list: List[int]
    D_local_list: List[int]
    input_split_sizes: List[int] = field(default_factory=list)
    output_split_sizes: List[int] = field(default_factory=list)
    codecs: Optional[QuantizedCommCodecs] = None


@dataclass
class ReduceScatterInfo:
    input_sizes: List[torch.Size]
    codecs: Optional[QuantizedCommCodecs] = None


@dataclass
class ReduceScatterBaseInfo:
    input_sizes: torch.Size
    codecs: Optional[QuantizedCommCodecs] = None


@dataclass
class AllGatherBaseInfo:
    input_size: torch.Size
    codecs: Optional[QuantizedCommCodecs] = None


@dataclass
class ReduceScatterVInfo:
    input_sizes: List[List[int]]
    input_splits: List[int]
    equal_splits: bool
    total_input_size: List[int]
    codecs: Optional[QuantizedCommCodecs] = None


def _encode(codecs, direction: str, t: Tensor, ctx=None) -> Tensor:
    if codecs is None:
        return t
    return getattr(codecs, direction).encode(t, ctx)


class _LazyCat:
    """Pieces of an uneven all-gather, concatenated only when the result is read."""

    def __init__(self, parts: List[Tensor]) -> None:
        self.parts = parts

    def materialize(self) -> Tensor:
        return torch.cat(self.parts, dim=0)


def _decode(codecs, direction: str, t, ctx=None) -> Tensor:
    if isinstance(t, _LazyCat):
        t = t.materialize()
    if codecs is None:
        return t
    return getattr(codecs, direction).decode(t, ctx)


def _chunk_ctx(codec, width: int):
    """Context of one destination's chunk: codecs that quantise by row and were given no row length use the chunk's row width."""
    ctx = codec.create_context()
    if ctx is not None and getattr(ctx, "row_dim", 1) <= 0:
        ctx.row_dim = int(width)
    return ctx


def _is_byte_codec(codec) -> bool:
    return codec.quantized_dtype == torch.uint8


def _encode_chunks(codec, flat: Tensor, elem_splits: List[int], widths: List[int]) -> Tuple[Tensor, List[int]]:
    """Encode what goes to every destination.  Cast codecs keep the element count and run once over the whole buffer; byte codecs
    (FP8 / INT8 / MX4 containers) run per destination so that no quantisation block straddles two destinations, and report the
    encoded split sizes."""
    if not _is_byte_codec(codec):
        return codec.encode(flat, codec.create_context()), [int(n) for n in elem_splits]
    parts = [codec.encode(c, _chunk_ctx(codec, w)) if c.numel() else flat.new_empty(0, dtype=torch.uint8) for c, w in zip(flat.split(elem_splits), widths)]
    return torch.cat(parts), [int(e.numel()) for e in parts]


def _encoded_sizes(codec, elem_splits: List[int], widths: List[int]) -> List[int]:
    if not _is_byte_codec(codec):
        return [int(n) for n in elem_splits]
    return [int(codec.calc_quantized_size(int(n), _chunk_ctx(codec, w))) if n else 0 for n, w in zip(elem_splits, widths)]


def _decode_chunks(codec, flat: Tensor, elem_splits: List[int], widths: List[int], out_dtype: torch.dtype) -> Tensor:
    """Inverse of :func:`_encode_chunks` for what arrived from every source."""
    if not _is_byte_codec(codec):
        ctx = codec.create_context()
        if ctx is not None:
            ctx.dtype = out_dtype
        return codec.decode(flat, ctx)
    out = []
    for part, n, w in zip(flat.split(_encoded_sizes(codec, elem_splits, widths)), elem_splits, widths):
        if n == 0:
            continue
        ctx = _chunk_ctx(codec, w)
        ctx.dtype = out_dtype
        ctx.numel = int(n)
        out.append(codec.decode(part, ctx)[: int(n)])
    return torch.cat(out) if out else flat.new_empty(0, dtype=out_dtype)


# ---- pooled all-to-all -----------------------------------------------------------------------------
def _recat_pooled_embedding_grad_out(grad_output: Tensor, num_features_per_rank: List[int]) -> Tensor:
    """``[B_local, sum(D_r)]`` -> flat buffer with rank r's ``[B_local, D_r]`` block contiguous."""
    grads = grad_output.split(num_features_per_rank, dim=1)
    return torch.cat([g.contiguous().view(-1) for g in grads], dim=0)


class All2All_Pooled_Req(Function):
    @staticmethod
    def forward(ctx, pg, myreq: Request, a2ai: All2AllPooledInfo, input_embeddings: Tensor) -> Tensor:
        my_rank = dist.get_rank(pg)
        (B_global, D_local_sum) = input_embeddings.shape
        dim_sum_per_rank = a2ai.dim_sum_per_rank
        batch_size_per_rank = a2ai.batch_size_per_rank
        B_local = batch_size_per_rank[my_rank]
        assert B_global == sum(batch_size_per_rank)
        sharded_input = input_embeddings.contiguous().view(-1)
        qctx = None
        input_split_sizes = [D_local_sum * b for b in batch_size_per_rank]
        output_split_sizes = [B_local * d for d in dim_sum_per_rank]
        a2ai.value_dtype = input_embeddings.dtype
        if a2ai.codecs is not None:
            sharded_input, input_split_sizes = _encode_chunks(a2ai.codecs.forward, sharded_input, input_split_sizes, [D_local_sum] * len(batch_size_per_rank))
            output_split_sizes = _encoded_sizes(a2ai.codecs.forward, output_split_sizes, dim_sum_per_rank)
        sharded_output = torch.empty(sum(output_split_sizes), dtype=sharded_input.dtype, device=sharded_input.device)
        with record_function("## alltoall_fwd_single ##"):
            req = _all_to_all_single(sharded_output, sharded_input, output_split_sizes, input_split_sizes, pg, async_op=True)
        myreq.req = req
        myreq.tensor = sharded_output
        myreq.qcomm_ctx = qctx
        myreq.info = a2ai
        myreq.wait_function = All2All_Pooled_Wait
        ctx.myreq = myreq
        ctx.pg = pg
        return myreq.dummy_tensor

    @staticmethod
    def backward(ctx, *unused):
        myreq: Request = ctx.myreq
        a2ai: All2AllPooledInfo = myreq.info
        myreq.req.wait()
        myreq.req = None
        grad_output = myreq.tensor
        my_rank = dist.get_rank(ctx.pg)
        D_local_sum = a2ai.dim_sum_per_rank[my_rank]
        if a2ai.codecs is not None:
            grad_output = _decode_chunks(a2ai.codecs.backward, grad_output, [D_local_sum * b for b in a2ai.batch_size_per_rank],
                                         [D_local_sum] * len(a2ai.batch_size_per_rank), getattr(a2ai, "grad_dtype", torch.float32))
        grad_input = grad_output.view(sum(a2ai.batch_size_per_rank), D_local_sum)
        if GRADIENT_DIVISION:
            grad_input = grad_input / dist.get_world_size(ctx.pg)
        myreq.tensor = None
        myreq.dummy_tensor = None
        return None, None, None, grad_input


class All2All_Pooled_Wait(Function):
    @staticmethod
    def forward(ctx, pg, myreq: Request, *dummy) -> Tensor:
        a2ai: All2AllPooledInfo = myreq.info
        ctx.a2ai = a2ai
        ctx.pg = pg
        ctx.myreq = myreq
        myreq.req.wait()
        sharded_output = myreq.tensor
        myreq.req = None
        myreq.tensor = None
        my_rank = dist.get_rank(pg)
        B_local = a2ai.batch_size_per_rank[my_rank]
        if a2ai.codecs is not None:
            sharded_output = _decode_chunks(a2ai.codecs.forward, sharded_output, [B_local * d for d in a2ai.dim_sum_per_rank], a2ai.dim_sum_per_rank,
                                            getattr(a2ai, "value_dtype", torch.float32))
        outputs = sharded_output.split([B_local * d for d in a2ai.dim_sum_per_rank])
        return torch.cat([o.view(B_local, -1) for o in outputs], dim=1)

    @staticmethod
    def backward(ctx, grad_output: Tensor):
        myreq: Request = ctx.myreq
        a2ai: All2AllPooledInfo = ctx.a2ai
        pg = ctx.pg
        my_rank = dist.get_rank(pg)
        B_local = a2ai.batch_size_per_rank[my_rank]
        D_local_sum = a2ai.dim_sum_per_rank[my_rank]
        sharded_grad_output = _recat_pooled_embedding_grad_out(grad_output.contiguous(), a2ai.dim_sum_per_rank)
        qctx = None
        input_split_sizes = [B_local * d for d in a2ai.dim_sum_per_rank]
        output_split_sizes = [D_local_sum * b for b in a2ai.batch_size_per_rank]
        a2ai.grad_dtype = grad_output.dtype
        if a2ai.codecs is not None:
            sharded_grad_output, input_split_sizes = _encode_chunks(a2ai.codecs.backward, sharded_grad_output, input_split_sizes, a2ai.dim_sum_per_rank)
            output_split_sizes = _encoded_sizes(a2ai.codecs.backward, output_split_sizes, [D_local_sum] * len(a2ai.batch_size_per_rank))
        sharded_grad_input = torch.empty(sum(output_split_sizes), device=sharded_grad_output.device, dtype=sharded_grad_output.dtype)
        with record_function("## alltoall_bwd_single ##"):
            req = _all_to_all_single(sharded_grad_input, sharded_grad_output, output_split_sizes, input_split_sizes, pg, async_op=True)
        myreq.req = req
        myreq.tensor = sharded_grad_input
        myreq.qcomm_ctx = qctx
        return None, None, myreq.dummy_tensor


def alltoall_pooled(
    a2a_pooled_embs_tensor: Tensor,
    batch_size_per_rank: List[int],
    dim_sum_per_rank: List[int],
    dim_sum_per_rank_tensor: Optional[Tensor] = None,
    cumsum_dim_sum_per_rank_tensor: Optional[Tensor] = None,
    group: Optional[dist.ProcessGroup] = None,
    codecs: Optional[QuantizedCommCodecs] = None,
) -> Awaitable[Tensor]:
    """``[B_global, D_local_sum]`` on every rank -> ``[B_local, sum_r D_r]``."""
    if group is None:
        group = dist.distributed_c10d._get_default_group()
    if dist.get_world_size(group) <= 1:
        return NoWait(a2a_pooled_embs_tensor)
    a2ai = All2AllPooledInfo(batch_size_per_rank, dim_sum_per_rank, dim_sum_per_rank_tensor, cumsum_dim_sum_per_rank_tensor, codecs)
    myreq = Request(group, device=a2a_pooled_embs_tensor.device)
    All2All_Pooled_Req.apply(group, myreq, a2ai, a2a_pooled_embs_tensor)
    return myreq


# ---- sequence all-to-all ---------------------------------------------------------------------------
class All2All_Seq_Req(Function):
    @staticmethod
    def forward(ctx, pg, myreq: Request, a2ai: All2AllSequenceInfo, sharded_input_embeddings: Tensor) -> Tensor:
        D = a2ai.embedding_dim
        forward_recat = a2ai.forward_recat_tensor
        lengths = a2ai.lengths_after_sparse_data_all2all * D
        local_T = lengths.shape[0] if lengths.dim() > 1 else None
        qctx = None
        if forward_recat is not None and lengths.numel() > 0 and not a2ai.variable_batch_size:
            # reorder (feature, source rank) -> (source rank, feature) so that each peer's rows are contiguous
            plen, sharded_input_embeddings, _ = sops.permute_2D_sparse_data(
                forward_recat, lengths.reshape(forward_recat.numel(), -1),
                sharded_input_embeddings.reshape(-1), None, sharded_input_embeddings.numel(),
            )
            a2ai.permuted_lengths_after_sparse_data_all2all = plen
        elif forward_recat is not None and lengths.numel() > 0:
            plen, sharded_input_embeddings, _ = sops.permute_1D_sparse_data(
                forward_recat, lengths.view(-1), sharded_input_embeddings.reshape(-1), None, sharded_input_embeddings.numel()
            )
            a2ai.permuted_lengths_after_sparse_data_all2all = plen
        del local_T
        a2ai.value_dtype = sharded_input_embeddings.dtype
        sharded_input_embeddings = sharded_input_embeddings.reshape(-1)
        # rows travel the routes of the ids in reverse: what the id all-to-all received from a peer is sent back to it
        out_splits = [s * D for s in a2ai.input_splits]
        in_splits = [s * D for s in a2ai.output_splits]
        if a2ai.codecs is not None:
            sharded_input_embeddings, in_splits = _encode_chunks(a2ai.codecs.forward, sharded_input_embeddings, in_splits, [D] * len(in_splits))
            out_splits = _encoded_sizes(a2ai.codecs.forward, out_splits, [D] * len(out_splits))
        sharded_output = torch.empty(sum(out_splits), dtype=sharded_input_embeddings.dtype, device=sharded_input_embeddings.device)
        with record_function("## alltoall_seq_embedding_fwd_single ##"):
            req = _all_to_all_single(sharded_output, sharded_input_embeddings, out_splits, in_splits, pg, async_op=True)
        myreq.req = req
        myreq.tensor = sharded_output
        myreq.info = a2ai
        myreq.qcomm_ctx = qctx
        myreq.wait_function = All2All_Seq_Req_Wait
        ctx.myreq = myreq
        ctx.pg = pg
        return myreq.dummy_tensor

    @staticmethod
    def backward(ctx, *unused):
        myreq: Request = ctx.myreq
        a2ai: All2AllSequenceInfo = myreq.info
        D = a2ai.embedding_dim
        myreq.req.wait()
        grad = myreq.tensor
        if a2ai.codecs is not None:
            splits = [s * D for s in a2ai.output_splits]
            grad = _decode_chunks(a2ai.codecs.backward, grad, splits, [D] * len(splits), getattr(a2ai, "grad_dtype", torch.float32))
        myreq.req = None
        myreq.tensor = None
        backward_recat = a2ai.backward_recat_tensor
        lengths = (a2ai.permuted_lengths_after_sparse_data_all2all if a2ai.permuted_lengths_after_sparse_data_all2all is not None else a2ai.lengths_after_sparse_data_all2all)
        if backward_recat is not None and lengths.numel() > 0:
            # the permuted lengths saved by forward are already in elements (rows * D)
            plen = lengths if a2ai.permuted_lengths_after_sparse_data_all2all is not None else lengths * D
            if a2ai.variable_batch_size:
                _, grad, _ = sops.permute_1D_sparse_data(backward_recat, plen.view(-1), grad.reshape(-1), None, grad.numel())
            else:
                _, grad, _ = sops.permute_2D_sparse_data(backward_recat, plen.reshape(backward_recat.numel(), -1), grad.reshape(-1), None, grad.numel())
        grad_input = grad.view(-1, D)
        if GRADIENT_DIVISION:
            grad_input = grad_input / dist.get_world_size(ctx.pg)
        myreq.dummy_tensor = None
        return None, None, None, grad_input


class All2All_Seq_Req_Wait(Function):
    @staticmethod
    def forward(ctx, pg, myreq: Request, *dummy) -> Tensor:
        a2ai: All2AllSequenceInfo = myreq.info
        ctx.a2ai = a2ai
        ctx.pg = pg
        ctx.myreq = myreq
        myreq.req.wait()
        out = myreq.tensor
        if a2ai.codecs is not None:
            splits = [s * a2ai.embedding_dim for s in a2ai.input_splits]
            out = _decode_chunks(a2ai.codecs.forward, out, splits, [a2ai.embedding_dim] * len(splits), getattr(a2ai, "value_dtype", torch.float32))
        myreq.req = None
        myreq.tensor = None
        return out.view(-1, a2ai.embedding_dim)

    @staticmethod
    def backward(ctx, sharded_grad_output: Tensor):
        myreq: Request = ctx.myreq
        a2ai: All2AllSequenceInfo = ctx.a2ai
        D = a2ai.embedding_dim
        g = sharded_grad_output.contiguous().view(-1)
        qctx = None
        a2ai.grad_dtype = sharded_grad_output.dtype
        out_splits = [s * D for s in a2ai.output_splits]
        in_splits = [s * D for s in a2ai.input_splits]
        if a2ai.codecs is not None:
            g, in_splits = _encode_chunks(a2ai.codecs.backward, g, in_splits, [D] * len(in_splits))
            out_splits = _encoded_sizes(a2ai.codecs.backward, out_splits, [D] * len(out_splits))
        grad_input = torch.empty(sum(out_splits), device=g.device, dtype=g.dtype)
        with record_function("## alltoall_seq_embedding_bwd_single ##"):
            req = _all_to_all_single(grad_input, g, out_splits, in_splits, ctx.pg, async_op=True)
        myreq.req = req
        myreq.tensor = grad_input
        myreq.qcomm_ctx = qctx
        return None, None, myreq.dummy_tensor


def alltoall_sequence(
    a2a_sequence_embs_tensor: Tensor,
    forward_recat_tensor: Optional[Tensor],
    backward_recat_tensor: Tensor,
    lengths_after_sparse_data_all2all: Tensor,
    input_splits: List[int],
    output_splits: List[int],
    variable_batch_size: bool = False,
    group: Optional[dist.ProcessGroup] = None,
    codecs: Optional[QuantizedCommCodecs] = None,
) -> Awaitable[Tensor]:
    """Send each looked-up row ``[sum L, D]`` back to the rank that asked for it."""
    if group is None:
        group = dist.distributed_c10d._get_default_group()
    if dist.get_world_size(group) <= 1:
        return NoWait(a2a_sequence_embs_tensor)
    a2ai = All2AllSequenceInfo(
        embedding_dim=a2a_sequence_embs_tensor.shape[1],
        lengths_after_sparse_data_all2all=lengths_after_sparse_data_all2all,
        forward_recat_tensor=forward_recat_tensor,
        backward_recat_tensor=backward_recat_tensor,
        input_splits=input_splits,
        output_splits=output_splits,
        variable_batch_size=variable_batch_size,
        codecs=codecs,
    )
    if forward_recat_tensor is not None and lengths_after_sparse_data_all2all.numel() > 0:
        # lengths in the permuted (source rank, feature) order, needed to undo the permute in backward
        if variable_batch_size:
            a2ai.permuted_lengths_after_sparse_data_all2all = lengths_after_sparse_data_all2all.view(-1).index_select(0, forward_recat_tensor.to(torch.int64))
        else:
            a2ai.permuted_lengths_after_sparse_data_all2all = lengths_after_sparse_data_all2all.view(forward_recat_tensor.numel(), -1).index_select(0, forward_recat_tensor.to(torch.int64))
    myreq = Request(group, device=a2a_sequence_embs_tensor.device)
    All2All_Seq_Req.apply(group, myreq, a2ai, a2a_sequence_embs_tensor)
    return myreq


# ---- reduce-scatter (row-wise sharding) ------------------------------------------------------------
class ReduceScatterBase_Req(Function):
    @staticmethod
    def forward(ctx, pg, myreq: Request, rsi: ReduceScatterBaseInfo, inputs: Tensor) -> Tensor:
        W = dist.get_world_size(pg)
        qctx = None
        x = inputs.contiguous()
        if rsi.codecs is not None:
            qctx = rsi.codecs.forward.create_context()
            x = rsi.codecs.forward.encode(x, qctx)
        out = x.new_empty((x.shape[0] // W,) + tuple(x.shape[1:]))
        with record_function("## reduce_scatter_base ##"):
            req = _reduce_scatter_tensor(out, x, pg, async_op=True)
        myreq.req, myreq.tensor, myreq.info, myreq.qcomm_ctx = req, out, rsi, qctx
        myreq.wait_function = ReduceScatterBase_Wait
        ctx.myreq, ctx.pg = myreq, pg
        return myreq.dummy_tensor

    @staticmethod
    def backward(ctx, *unused):
        myreq: Request = ctx.myreq
        myreq.req.wait()
        grad = _decode(myreq.info.codecs, "backward", myreq.tensor, myreq.qcomm_ctx)
        myreq.req = None
        myreq.tensor = None
        if GRADIENT_DIVISION:
            grad = grad / dist.get_world_size(ctx.pg)
        myreq.dummy_tensor = None
        return None, None, None, grad


class ReduceScatterBase_Wait(Function):
    @staticmethod
    def forward(ctx, pg, myreq: Request, *dummy) -> Tensor:
        myreq.req.wait()
        out = _decode(myreq.info.codecs, "forward", myreq.tensor, myreq.qcomm_ctx)
        myreq.req = None
        myreq.tensor = None
        ctx.myreq, ctx.pg = myreq, pg
        return out

    @staticmethod
    def backward(ctx, grad_output: Tensor):
        myreq: Request = ctx.myreq
        rsi = myreq.info
        g = grad_output.contiguous()
        qctx = None
        if rsi.codecs is not None:
            qctx = rsi.codecs.backward.create_context()
            g = rsi.codecs.backward.encode(g, qctx)
        W = dist.get_world_size(ctx.pg)
        grad_inputs = g.new_empty((g.shape[0] * W,) + tuple(g.shape[1:]))
        with record_function("## reduce_scatter_base_bw (all_gather) ##"):
            req = _all_gather_into_tensor(grad_inputs, g, ctx.pg, async_op=True)
        myreq.req, myreq.tensor, myreq.qcomm_ctx = req, grad_inputs, qctx
        return None, None, myreq.dummy_tensor


def reduce_scatter_base_pooled(inputs: Tensor, group: Optional[dist.ProcessGroup] = None, codecs: Optional[QuantizedCommCodecs] = None) -> Awaitable[Tensor]:
    """``[W*B, D]`` partial sums on every rank -> ``[B, D]`` summed, rank r keeping rows ``[r*B, (r+1)*B)``."""
    if group is None:
        group = dist.distributed_c10d._get_default_group()
    if dist.get_world_size(group) <= 1:
        return NoWait(inputs)
    rsi = ReduceScatterBaseInfo(input_sizes=inputs.size(), codecs=codecs)
    myreq = Request(group, device=inputs.device)
    ReduceScatterBase_Req.apply(group, myreq, rsi, inputs)
    return myreq


def reduce_scatter_pooled(inputs: List[Tensor], group: Optional[dist.ProcessGroup] = None, codecs: Optional[QuantizedCommCodecs] = None) -> Awaitable[Tensor]:
    """List form: ``inputs[r]`` is this rank's contribution to rank r."""
    if group is None:
        group = dist.distributed_c10d._get_default_group()
    if dist.get_world_size(group) <= 1:
        return NoWait(inputs[dist.get_rank(group)])
    sizes = {tuple(t.shape) for t in inputs}
    if len(sizes) == 1:
        return reduce_scatter_base_pooled(torch.cat(inputs, dim=0), group, codecs)
    return reduce_scatter_v_pooled(torch.cat(inputs, dim=0), [t.shape[0] for t in inputs], group, codecs)


class ReduceScatterV_Req(Function):
    @staticmethod
    def forward(ctx, pg, myreq: Request, rsi: ReduceScatterVInfo, inp: Tensor) -> Tensor:
        rank = dist.get_rank(pg)
        x = inp.contiguous()
        qctx = None
        if rsi.codecs is not None:
            qctx = rsi.codecs.forward.create_context()
            x = rsi.codecs.forward.encode(x, qctx)
        out = x.new_empty((rsi.input_splits[rank],) + tuple(x.shape[1:]))
        with record_function("## reduce_scatter_v ##"):
            req = _reduce_scatter_v(out, x, rsi.input_splits, pg, async_op=True)
        myreq.req, myreq.tensor, myreq.info, myreq.qcomm_ctx = req, out, rsi, qctx
        myreq.wait_function = ReduceScatterV_Wait
        ctx.myreq, ctx.pg = myreq, pg
        return myreq.dummy_tensor

    @staticmethod
    def backward(ctx, *unused):
        myreq: Request = ctx.myreq
        myreq.req.wait()
        grad = _decode(myreq.info.codecs, "backward", myreq.tensor, myreq.qcomm_ctx)
        myreq.req = None
        myreq.tensor = None
        if GRADIENT_DIVISION:
            grad = grad / dist.get_world_size(ctx.pg)
        myreq.dummy_tensor = None
        return None, None, None, grad


class ReduceScatterV_Wait(Function):
    @staticmethod
    def forward(ctx, pg, myreq: Request, *dummy) -> Tensor:
        myreq.req.wait()
        out = _decode(myreq.info.codecs, "forward", myreq.tensor, myreq.qcomm_ctx)
        myreq.req = None
        myreq.tensor = None
        ctx.myreq, ctx.pg = myreq, pg
        return out

    @staticmethod
    def backward(ctx, grad_output: Tensor):
        myreq: Request = ctx.myreq
        rsi: ReduceScatterVInfo = myreq.info
        g = grad_output.contiguous()
        qctx = None
        if rsi.codecs is not None:
            qctx = rsi.codecs.backward.create_context()
            g = rsi.codecs.backward.encode(g, qctx)
        outs = [g.new_empty((n,) + tuple(g.shape[1:])) for n in rsi.input_splits]
        with record_function("## reduce_scatter_v_bw (all_gather_v) ##"):
            req = dist.all_gather(outs, g, group=ctx.pg, async_op=True)

        class _Cat:
            def __init__(self, r, outs):
                self.r, self.outs = r, outs

            def wait(self):
                self.r.wait()

        myreq.req = _Cat(req, outs)
        myreq.tensor = _LazyCat(outs)
        myreq.qcomm_ctx = qctx
        return None, None, myreq.dummy_tensor


def reduce_scatter_v_pooled(inp: Tensor, input_splits: List[int], group: Optional[dist.ProcessGroup] = None, codecs: Optional[QuantizedCommCodecs] = None) -> Awaitable[Tensor]:
    """Reduce-scatter with a different number of rows per rank (variable batch per rank)."""
    if group is None:
        group = dist.distributed_c10d._get_default_group()
    if dist.get_world_size(group) <= 1:
        return NoWait(inp)
    rsi = ReduceScatterVInfo(
        input_sizes=[[s] + list(inp.shape[1:]) for s in input_splits], input_splits=input_splits,
        equal_splits=all(s == input_splits[0] for s in input_splits), total_input_size=list(inp.size()), codecs=codecs,
    )
    myreq = Request(group, device=inp.device)
    ReduceScatterV_Req.apply(group, myreq, rsi, inp)
    return myreq


# ---- all-gather (backward of reduce-scatter, also used by row-wise sequence paths) -----------------
class AllGatherBase_Req(Function):
    @staticmethod
    def forward(ctx, pg, myreq: Request, agi: AllGatherBaseInfo, inp: Tensor) -> Tensor:
        W = dist.get_world_size(pg)
        x = inp.contiguous()
        qctx = None
        if agi.codecs is not None:
            qctx = agi.codecs.forward.create_context()
            x = agi.codecs.forward.encode(x, qctx)
        out = x.new_empty((x.shape[0] * W,) + tuple(x.shape[1:]))
        with record_function("## all_gather_base ##"):
            req = _all_gather_into_tensor(out, x, pg, async_op=True)
        myreq.req, myreq.tensor, myreq.info, myreq.qcomm_ctx = req, out, agi, qctx
        myreq.wait_function = AllGatherBase_Wait
        ctx.myreq, ctx.pg = myreq, pg
        return myreq.dummy_tensor

    @staticmethod
    def backward(ctx, *unused):
        myreq: Request = ctx.myreq
        myreq.req.wait()
        grad = _decode(myreq.info.codecs, "backward", myreq.tensor, myreq.qcomm_ctx)
        myreq.req = None
        myreq.tensor = None
        if GRADIENT_DIVISION:
            grad = grad / dist.get_world_size(ctx.pg)
        myreq.dummy_tensor = None
        return None, None, None, grad


class AllGatherBase_Wait(Function):
    @staticmethod
    def forward(ctx, pg, myreq: Request, *dummy) -> Tensor:
        myreq.req.wait()
        out = _decode(myreq.info.codecs, "forward", myreq.tensor, myreq.qcomm_ctx)
        myreq.req = None
        myreq.tensor = None
        ctx.myreq, ctx.pg = myreq, pg
        return out

    @staticmethod
    def backward(ctx, grad_outputs: Tensor):
        myreq: Request = ctx.myreq
        agi = myreq.info
        g = grad_outputs.contiguous()
        qctx = None
        if agi.codecs is not None:
            qctx = agi.codecs.backward.create_context()
            g = agi.codecs.backward.encode(g, qctx)
        W = dist.get_world_size(ctx.pg)
        grad_input = g.new_empty((g.shape[0] // W,) + tuple(g.shape[1:]))
        with record_function("## all_gather_base_bw (reduce_scatter) ##"):
            req = _reduce_scatter_tensor(grad_input, g, ctx.pg, async_op=True)
        myreq.req, myreq.tensor, myreq.qcomm_ctx = req, grad_input, qctx
        return None, None, myreq.dummy_tensor


def all_gather_base_pooled(inp: Tensor, group: Optional[dist.ProcessGroup] = None, codecs: Optional[QuantizedCommCodecs] = None) -> Awaitable[Tensor]:
    """``[B, D]`` on every rank -> ``[W*B, D]``; gradient is reduce-scattered."""
    if group is None:
        group = dist.distributed_c10d._get_default_group()
    if dist.get_world_size(group) <= 1:
        return NoWait(inp)
    agi = AllGatherBaseInfo(input_size=inp.size(), codecs=codecs)
    myreq = Request(group, device=inp.device)
    AllGatherBase_Req.apply(group, myreq, agi, inp)
    return myreq


# ---- variable-batch pooled all-to-all (variable batch per feature) -----------------------------------
class Variable_Batch_All2All_Pooled(Function):
    """Synchronous autograd collective for the variable-batch-per-feature pooled output: every
    (rank, feature) block has its own batch size, so the payload is a flat 1-D buffer."""

    @staticmethod
    def forward(ctx, pg, a2ai: VariableBatchAll2AllPooledInfo, x: Tensor) -> Tensor:
        my_rank = dist.get_rank(pg)
        W = dist.get_world_size(pg)
        local_dims = a2ai.emb_dim_per_rank_per_feature[my_rank]
        in_splits = [sum(b * d for b, d in zip(a2ai.batch_size_per_rank_per_feature[r], local_dims)) for r in range(W)]
        out_splits = [
            sum(b * d for b, d in zip(a2ai.batch_size_per_feature_pre_a2a[sum(len(e) for e in a2ai.emb_dim_per_rank_per_feature[:r]):][: len(a2ai.emb_dim_per_rank_per_feature[r])], a2ai.emb_dim_per_rank_per_feature[r]))
            for r in range(W)
        ]
        a2ai.input_splits, a2ai.output_splits = in_splits, out_splits
        qctx = None
        xin = x.contiguous().view(-1)
        if a2ai.codecs is not None:
            qctx = a2ai.codecs.forward.create_context()
            xin = a2ai.codecs.forward.encode(xin, qctx)
        out = torch.empty(sum(out_splits), dtype=xin.dtype, device=xin.device)
        _all_to_all_single(out, xin, out_splits, in_splits, pg, async_op=False)
        ctx.pg, ctx.a2ai = pg, a2ai
        return _decode(a2ai.codecs, "forward", out, qctx)

    @staticmethod
    def backward(ctx, grad: Tensor):
        a2ai = ctx.a2ai
        g = grad.contiguous().view(-1)
        qctx = None
        if a2ai.codecs is not None:
            qctx = a2ai.codecs.backward.create_context()
            g = a2ai.codecs.backward.encode(g, qctx)
        out = torch.empty(sum(a2ai.input_splits), dtype=g.dtype, device=g.device)
        _all_to_all_single(out, g, a2ai.input_splits, a2ai.output_splits, ctx.pg, async_op=False)
        out = _decode(a2ai.codecs, "backward", out, qctx)
        if GRADIENT_DIVISION:
            out = out / dist.get_world_size(ctx.pg)
        return None, None, out


def variable_batch_alltoall_pooled(
    a2a_pooled_embs_tensor: Tensor,
    batch_size_per_rank_per_feature: List[List[int]],
    batch_size_per_feature_pre_a2a: List[int],
    emb_dim_per_rank_per_feature: List[List[int]],
    group: Optional[dist.ProcessGroup] = None,
    codecs: Optional[QuantizedCommCodecs] = None,
) -> Awaitable[Tensor]:
    if group is None:
        group = dist.distributed_c10d._get_default_group()
    if dist.get_world_size(group) <= 1:
        return NoWait(a2a_pooled_embs_tensor)
    a2ai = VariableBatchAll2AllPooledInfo(batch_size_per_rank_per_feature, batch_size_per_feature_pre_a2a, emb_dim_per_rank_per_feature, codecs)
    return NoWait(Variable_Batch_All2All_Pooled.apply(group, a2ai, a2a_pooled_embs_tensor))


# ---- generic tensor all-to-all (object pools) --------------------------------------------------------
class _TensorAllToAll(Function):
    @staticmethod
    def forward(ctx, pg, x: Tensor, in_splits: List[int], out_splits: List[int]) -> Tensor:
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        _all_to_all_single(out, x.contiguous(), out_splits, in_splits, pg, async_op=False)
        ctx.pg, ctx.in_splits, ctx.out_splits = pg, in_splits, out_splits
        return out

    @staticmethod
    def backward(ctx, g: Tensor):
        out = g.new_empty((sum(ctx.in_splits),) + tuple(g.shape[1:]))
        _all_to_all_single(out, g.contiguous(), ctx.in_splits, ctx.out_splits, ctx.pg, async_op=False)
        return None, out, None, None


def tensor_alltoall(x: Tensor, in_splits: List[int], out_splits: List[int], group: Optional[dist.ProcessGroup] = None) -> Tensor:
    """Differentiable ``all_to_all_single`` over dim 0."""
    if group is None:
        group = dist.distributed_c10d._get_default_group()
    if dist.get_world_size(group) <= 1:
        return x
    return _TensorAllToAll.apply(group, x, in_splits, out_splits)


# --------------------------------------------------------------------------------------
# Blocking forms: the same collectives with the result returned directly.  Code that cannot hold an ``Awaitable`` (a traced or
# exported region, a debugging session) switches to them with ``set_use_sync_collectives(True)``; they stay differentiable because
# they run the request / wait functions above back to back.  (``torchrec/distributed/comm_ops.py:1090-1600`` of the reference.)
# --------------------------------------------------------------------------------------
def torchrec_use_sync_collectives() -> bool:
    return get_use_sync_collectives()


def pg_name(pg: dist.ProcessGroup) -> str:
    """The registered name of a process group (what functional collectives take instead of the object)."""
    return dist._functional_collectives._resolve_group_name(pg, "") if hasattr(dist, "_functional_collectives") else str(pg)


def all2all_pooled_sync(pg: dist.ProcessGroup, a2ai: All2AllPooledInfo, input_embeddings: Tensor) -> Tensor:
    return alltoall_pooled(input_embeddings, a2ai.batch_size_per_rank, a2ai.dim_sum_per_rank, a2ai.dim_sum_per_rank_tensor, a2ai.cumsum_dim_sum_per_rank_tensor,
                           group=pg, codecs=a2ai.codecs).wait()


def variable_batch_all2all_pooled_sync(pg: dist.ProcessGroup, a2ai: VariableBatchAll2AllPooledInfo, input_embeddings: Tensor) -> Tensor:
    return variable_batch_alltoall_pooled(input_embeddings, a2ai.batch_size_per_rank_per_feature, a2ai.batch_size_per_feature_pre_a2a,
                                          a2ai.emb_dim_per_rank_per_feature, group=pg, codecs=a2ai.codecs).wait()


def all2all_sequence_sync(pg: dist.ProcessGroup, a2ai: All2AllSequenceInfo, sharded_input_embeddings: Tensor) -> Tensor:
    return alltoall_sequence(sharded_input_embeddings, a2ai.forward_recat_tensor, a2ai.backward_recat_tensor, a2ai.lengths_after_sparse_data_all2all,
                             a2ai.input_splits, a2ai.output_splits, a2ai.variable_batch_size, group=pg, codecs=a2ai.codecs).wait()


def reduce_scatter_sync(pg: dist.ProcessGroup, rsi: ReduceScatterInfo, *inputs: Tensor) -> Tensor:
    return reduce_scatter_pooled(list(inputs), group=pg, codecs=rsi.codecs).wait()


def reduce_scatter_base_sync(pg: dist.ProcessGroup, rsi: ReduceScatterBaseInfo, inputs: Tensor) -> Tensor:
    return reduce_scatter_base_pooled(inputs, group=pg, codecs=rsi.codecs).wait()


def all_gather_base_sync(pg: dist.ProcessGroup, agi: AllGatherBaseInfo, input: Tensor) -> Tensor:
    return all_gather_base_pooled(input, group=pg, codecs=agi.codecs).wait()


def reduce_scatter_v_sync(pg: dist.ProcessGroup, rsi: ReduceScatterVInfo, input: Tensor) -> Tensor:
    return reduce_scatter_v_pooled(input, list(rsi.input_splits), group=pg, codecs=rsi.codecs).wait()


def reduce_scatter_v_per_feature_pooled(input: Tensor, batch_size_per_rank_per_feature: List[List[int]], embedding_dims: List[int],
                                        group: Optional[dist.ProcessGroup] = None, codecs: Optional[QuantizedCommCodecs] = None) -> Awaitable[Tensor]:
    """Reduce-scatter of a flat pooled payload whose chunk for rank ``r`` holds, feature after feature, ``batch[r][f] * dim[f]`` values
    (features differ in batch size)."""
    if group is None:
        group = dist.distributed_c10d._get_default_group()
    if dist.get_world_size(group) <= 1:
        return NoWait(input)
    splits = [sum(b * d for b, d in zip(per_feature, embedding_dims)) for per_feature in batch_size_per_rank_per_feature]
    return reduce_scatter_v_pooled(input.view(-1), splits, group, codecs=codecs)


AllToAllSingle = _TensorAllToAll  # differentiable ``all_to_all_single`` over dim 0: ``apply(pg, x, in_splits, out_splits)``


class _AllGatherIntoTensor(Function):
    @staticmethod
    def forward(ctx, pg, shard: Tensor, gather_dim: int) -> Tensor:
        world = dist.get_world_size(pg)
        moved = shard.movedim(gather_dim, 0).contiguous()
        out = moved.new_empty((world * moved.shape[0],) + tuple(moved.shape[1:]))
        _all_gather_into_tensor(out, moved, pg, async_op=False)
        ctx.pg, ctx.dim = pg, gather_dim
        return out.movedim(0, gather_dim) if gather_dim else out

    @staticmethod
    def backward(ctx, g: Tensor):
        world = dist.get_world_size(ctx.pg)
        moved = g.movedim(ctx.dim, 0).contiguous()
        out = moved.new_empty((moved.shape[0] // world,) + tuple(moved.shape[1:]))
        _reduce_scatter_tensor(out, moved, ctx.pg, async_op=False)
        return None, (out.movedim(0, ctx.dim) if ctx.dim else out), None


class _ReduceScatterTensor(Function):
    @staticmethod
    def forward(ctx, pg, x: Tensor, scatter_dim: int) -> Tensor:
        world = dist.get_world_size(pg)
        moved = x.movedim(scatter_dim, 0).contiguous()
        out = moved.new_empty((moved.shape[0] // world,) + tuple(moved.shape[1:]))
        _reduce_scatter_tensor(out, moved, pg, async_op=False)
        ctx.pg, ctx.dim = pg, scatter_dim
        return out.movedim(0, scatter_dim) if scatter_dim else out

    @staticmethod
    def backward(ctx, g: Tensor):
        world = dist.get_world_size(ctx.pg)
        moved = g.movedim(ctx.dim, 0).contiguous()
        out = moved.new_empty((world * moved.shape[0],) + tuple(moved.shape[1:]))
        _all_gather_into_tensor(out, moved, ctx.pg, async_op=False)
        return None, (out.movedim(0, ctx.dim) if ctx.dim else out), None


def all_gather_into_tensor(shard: Tensor, gather_dim: int = 0, group: Optional[dist.ProcessGroup] = None) -> Tensor:
    """Differentiable all-gather along ``gather_dim`` (backward: reduce-scatter of the gradient)."""
    group = group if group is not None else dist.distributed_c10d._get_default_group()
    return shard if dist.get_world_size(group) <= 1 else _AllGatherIntoTensor.apply(group, shard, gather_dim)


def reduce_scatter_tensor(input: Tensor, scatter_dim: int = 0, group: Optional[dist.ProcessGroup] = None) -> Tensor:
    """Differentiable sum reduce-scatter along ``scatter_dim`` (backward: all-gather of the gradient)."""
    group = group if group is not None else dist.distributed_c10d._get_default_group()
    return input if dist.get_world_size(group) <= 1 else _ReduceScatterTensor.apply(group, input, scatter_dim)
