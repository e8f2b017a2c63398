"""Jagged / sparse-input operators.

Every function has two implementations:

* a composite one written with plain torch ops.  It runs on any device, is the CPU path
  (gloo tests, config without a GPU) and is the numerical oracle of the CUDA kernel;
* a hand-written sm_100a kernel in ``torchrec_b200/csrc/cuda/sparse_kernels.cu`` reached
  through ``torch.ops.trb200.*`` whenever the input lives on a CUDA device.

The reference calls the equivalent ``torch.ops.fbgemm.*`` operators of an external wheel
(call sites: ``torchrec/sparse/jagged_tensor.py:80,455,471,2577``;
``torchrec/distributed/embedding_sharding.py:263``; ``torchrec/distributed/dist_data.py:137``).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from . import _ext

# Ops whose CUDA kernel exists in the library.  Filled by name so that a kernel can be
# turned off for an A/B measurement with TRB200_COMPOSITE=<op,op,...>.
import os

_COMPOSITE_ONLY = set(filter(None, os.environ.get("TRB200_COMPOSITE", "").split(",")))


def _kern(t: torch.Tensor, name: str) -> bool:
    if name in _COMPOSITE_ONLY:
        return False
    return _ext.use_cuda_kernel(t, name)


def _cpu_native(name: str, *tensors: Optional[torch.Tensor]) -> bool:
    """Host tensors that take no part in autograd go to the C++ implementation (``csrc/cpu/sparse_cpu.cpp``) when the host
    library is built; the composite implementation stays the oracle and the differentiable path."""
    if name in _COMPOSITE_ONLY or os.environ.get("TRB200_CPU_NATIVE", "1") == "0":
        return False
    for t in tensors:
        if t is not None and (t.device.type != "cpu" or t.requires_grad):
            return False
    return _ext.has_cpu_ext()


# --------------------------------------------------------------------------------------
# scans
# --------------------------------------------------------------------------------------
def asynchronous_complete_cumsum(x: torch.Tensor) -> torch.Tensor:
    """``[n] -> [n+1]`` exclusive+total prefix sum (``out[0]=0, out[i+1]=sum(x[:i+1])``).

    A 2-D input ``[r, n]`` is scanned along dim 1 and returns ``[r, n+1]``.
    """
    if x.dim() == 1 and x.numel() > 0 and _kern(x, "complete_cumsum"):
        return torch.ops.trb200.complete_cumsum(x)
    if x.dim() == 1:
        out = x.new_zeros(x.numel() + 1)
        if x.numel():
            torch.cumsum(x, 0, out=out[1:])
        return out
    out = x.new_zeros(x.shape[0], x.shape[1] + 1)
    if x.numel():
        out[:, 1:] = torch.cumsum(x, 1)
    return out


def asynchronous_inclusive_cumsum(x: torch.Tensor) -> torch.Tensor:
    return torch.cumsum(x, 0).to(x.dtype)


def asynchronous_exclusive_cumsum(x: torch.Tensor) -> torch.Tensor:
    return asynchronous_complete_cumsum(x)[:-1]


def offsets_range(offsets: torch.Tensor, range_size: int) -> torch.Tensor:
    """``arange`` restarting at every segment start: position of each element in its bag.

    ``offsets`` are the segment starts ``[n]`` (no trailing total), ``range_size`` the
    total number of elements.
    """
    if range_size == 0:
        return offsets.new_empty(0)
    if offsets.dtype in (torch.int32, torch.int64) and offsets.numel() > 0 and _kern(offsets, "offsets_range"):
        return torch.ops.trb200.offsets_range(offsets.contiguous(), int(range_size))
    starts = offsets.to(torch.int64)
    ends = torch.cat([starts[1:], starts.new_tensor([range_size])])
    lens = ends - starts
    seg_start = torch.repeat_interleave(starts, lens, output_size=range_size)
    return (torch.arange(range_size, device=offsets.device) - seg_start).to(offsets.dtype)


def segment_sum_csr(batch_size: int, csr_seg: torch.Tensor, values: torch.Tensor) -> torch.Tensor:
    """``out[i] = sum(values[csr_seg[i]*batch_size : csr_seg[i+1]*batch_size])``."""
    n = csr_seg.numel() - 1
    if n <= 0:
        return values.new_zeros(0)
    if csr_seg.dtype in (torch.int32, torch.int64) and not values.requires_grad and _kern(values, "segment_sum_csr"):
        return torch.ops.trb200.segment_sum_csr(int(batch_size), csr_seg.contiguous(), values.reshape(-1).contiguous())
    cs = asynchronous_complete_cumsum(values.reshape(-1))
    idx = csr_seg.to(torch.int64) * batch_size
    return (cs[idx[1:]] - cs[idx[:-1]]).to(values.dtype)


def lengths_range(lengths: torch.Tensor, total: Optional[int] = None) -> torch.Tensor:
    """Segment id of every element given segment lengths (``repeat_interleave(arange)``)."""
    n = lengths.numel()
    ar = torch.arange(n, device=lengths.device)
    if total is None:
        return torch.repeat_interleave(ar, lengths.to(torch.int64))
    return torch.repeat_interleave(ar, lengths.to(torch.int64), output_size=total)


# --------------------------------------------------------------------------------------
# permutes
# --------------------------------------------------------------------------------------
def _permute_segments(
    values: torch.Tensor,
    seg_lengths: torch.Tensor,
    permute: torch.Tensor,
    weights: Optional[torch.Tensor],
    out_total: Optional[int],
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Move variable-length segments of ``values`` into the order given by ``permute``."""
    p = permute.to(torch.int64)
    seg_lengths = seg_lengths.to(torch.int64)
    in_off = asynchronous_complete_cumsum(seg_lengths)
    out_len = seg_lengths.index_select(0, p)
    out_off = asynchronous_complete_cumsum(out_len)
    if out_total is None:
        out_total = int(out_off[-1].item())
    if out_total == 0:
        return values.new_empty((0,) + tuple(values.shape[1:])), (
            None if weights is None else weights.new_empty((0,) + tuple(weights.shape[1:]))
        )
    seg_id = lengths_range(out_len, out_total)
    shift = in_off.index_select(0, p) - out_off[:-1]
    src = shift.index_select(0, seg_id) + torch.arange(out_total, device=values.device)
    out_v = values.index_select(0, src)
    out_w = None if weights is None else weights.index_select(0, src)
    return out_v, out_w


def permute_2D_sparse_data(
    permute: torch.Tensor,
    lengths: torch.Tensor,
    values: torch.Tensor,
    weights: Optional[torch.Tensor] = None,
    permuted_lengths_sum: Optional[int] = None,
) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """Reorder the rows of ``lengths [T, B]`` by ``permute [T']`` and move the matching
    value segments.  ``permute`` may repeat or drop rows."""
    assert lengths.dim() == 2
    if values.is_cuda and values.numel() > 0 and _kern(values, "permute_2D_sparse_data") and values.dim() == 1:
        return torch.ops.trb200.permute_2d_sparse_data(
            permute, lengths, values, weights, -1 if permuted_lengths_sum is None else int(permuted_lengths_sum)
        )
    if values.numel() > 0 and lengths.dtype in (torch.int32, torch.int64) and _cpu_native("permute_2D_sparse_data", values, weights, lengths):
        return _ext.cpu_ops().permute_2d_sparse_data(permute, lengths, values, weights)
    T, B = lengths.shape
    p = permute.to(torch.int64)
    out_lengths = lengths.index_select(0, p)
    row_tot = lengths.sum(1)
    out_v, out_w = _permute_segments(values, row_tot, p, weights, permuted_lengths_sum)
    return out_lengths, out_v, out_w


def permute_1D_sparse_data(
    permute: torch.Tensor,
    lengths: torch.Tensor,
    values: torch.Tensor,
    weights: Optional[torch.Tensor] = None,
    permuted_lengths_sum: Optional[int] = None,
) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """Same as :func:`permute_2D_sparse_data` with one length per segment."""
    p = permute.to(torch.int64)
    out_lengths = lengths.index_select(0, p)
    out_v, out_w = _permute_segments(values, lengths, p, weights, permuted_lengths_sum)
    return out_lengths, out_v, out_w


def invert_permute(permute: torch.Tensor) -> torch.Tensor:
    inv = torch.empty_like(permute)
    inv[permute.to(torch.int64)] = torch.arange(permute.numel(), device=permute.device, dtype=permute.dtype)
    return inv


def expand_into_jagged_permute(
    permute: torch.Tensor, input_offsets: torch.Tensor, output_offsets: torch.Tensor, output_size: int
) -> torch.Tensor:
    """Expand a segment permutation into an element permutation.

    Segment ``i`` of the output is segment ``permute[i]`` of the input; the result lists, for
    each output element, the index of its source element.
    """
    p = permute.to(torch.int64)
    in_off = input_offsets.to(torch.int64)
    out_off = output_offsets.to(torch.int64)
    out_len = out_off[1:] - out_off[:-1]
    seg_id = lengths_range(out_len, output_size)
    shift = in_off[:-1].index_select(0, p) - out_off[:-1]
    return (shift.index_select(0, seg_id) + torch.arange(output_size, device=permute.device)).to(permute.dtype)


def keyed_jagged_index_select_dim1(
    values: torch.Tensor,
    lengths: torch.Tensor,
    offsets: torch.Tensor,
    indices: torch.Tensor,
    batch_size: int,
    weights: Optional[torch.Tensor] = None,
    selected_lengths_sum: Optional[int] = None,
) -> List[torch.Tensor]:
    """Select the bags ``indices`` of every key of a ``[F, batch_size]`` jagged layout."""
    F = lengths.numel() // batch_size
    idx = indices.to(torch.int64)
    sel = (torch.arange(F, device=lengths.device).view(-1, 1) * batch_size + idx.view(1, -1)).reshape(-1)
    out_lengths = lengths.index_select(0, sel)
    out_v, out_w = _permute_segments(values, lengths, sel, weights, selected_lengths_sum)
    res = [out_v, out_lengths]
    if weights is not None:
        res.append(out_w)
    return res


def jagged_index_select(values: torch.Tensor, lengths: torch.Tensor, indices: torch.Tensor):
    """Select whole segments of a jagged ``values [N, ...]`` by segment index."""
    out_lengths = lengths.index_select(0, indices.to(torch.int64))
    out_v, _ = _permute_segments(values, lengths, indices, None, None)
    return out_v, out_lengths


# --------------------------------------------------------------------------------------
# row-wise bucketization
# --------------------------------------------------------------------------------------
def block_bucketize_sparse_features(
    lengths: torch.Tensor,
    indices: torch.Tensor,
    bucketize_pos: bool,
    sequence: bool,
    block_sizes: torch.Tensor,
    my_size: int,
    weights: Optional[torch.Tensor] = None,
    batch_size_per_feature: Optional[torch.Tensor] = None,
    max_B: int = -1,
    block_bucketize_pos: Optional[List[torch.Tensor]] = None,
    keep_orig_idx: bool = False,
    total_num_blocks: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor], Optional[torch.Tensor]]:
    """Split every bag of a ``[F, B]`` jagged input into ``my_size`` buckets by row block.

    For feature ``f`` an id goes to bucket ``id // block_sizes[f]`` and becomes the
    shard-local id ``id % block_sizes[f]`` (ids past ``block*my_size`` wrap:
    bucket ``id % my_size``, local id ``id // my_size``).  Output lengths are laid out
    ``[my_size, F, B]`` and ids bucket-major, keeping the original order inside a bag.

    Returns ``(new_lengths, new_indices, new_weights, new_pos, unbucketize_permute)``;
    ``new_pos`` is the position of the id in its original bag (``bucketize_pos``) and
    ``unbucketize_permute[i]`` the output slot of input element ``i`` (``sequence``).
    """
    if (
        indices.is_cuda
        and batch_size_per_feature is None
        and block_bucketize_pos is None
        and total_num_blocks is None
        and _kern(indices, "block_bucketize_sparse_features")
    ):
        return torch.ops.trb200.block_bucketize(
            lengths, indices, bucketize_pos, sequence, block_sizes, my_size, weights, keep_orig_idx
        )
    if (
        batch_size_per_feature is None and block_bucketize_pos is None and total_num_blocks is None and block_sizes.numel() > 0
        and lengths.dtype in (torch.int32, torch.int64) and indices.dtype in (torch.int32, torch.int64)
        and (weights is None or weights.dtype == torch.float32)
        and _cpu_native("block_bucketize_sparse_features", indices, lengths, weights)
    ):
        return _ext.cpu_ops().block_bucketize(lengths, indices, bucketize_pos, sequence, block_sizes, my_size, weights, keep_orig_idx)
    n_bags = lengths.numel()
    F = block_sizes.numel()
    N = indices.numel()
    dev = indices.device
    len64 = lengths.to(torch.int64)
    bag_id = lengths_range(len64, N)
    if batch_size_per_feature is not None:
        bpf = batch_size_per_feature.to(torch.int64)
        feat_of_bag = lengths_range(bpf, n_bags)
    else:
        B = n_bags // max(F, 1)
        feat_of_bag = torch.arange(n_bags, device=dev) // max(B, 1)
    feat = feat_of_bag.index_select(0, bag_id) if N else bag_id
    idx64 = indices.to(torch.int64)
    blk = block_sizes.to(torch.int64).index_select(0, feat) if N else idx64
    if block_bucketize_pos is not None:
        bucket = torch.empty_like(idx64)
        local = torch.empty_like(idx64)
        for f in range(F):
            m = feat == f
            bounds = block_bucketize_pos[f].to(torch.int64).to(dev)
            b = torch.bucketize(idx64[m], bounds, right=True) - 1
            b = b.clamp_(0, my_size - 1)
            bucket[m] = b
            local[m] = idx64[m] - bounds[b]
    else:
        if total_num_blocks is not None:
            tnb = total_num_blocks.to(torch.int64).index_select(0, feat) if N else idx64
            blocks_per_rank = tnb // my_size
            in_range = idx64 < blk * tnb
            bucket = torch.where(in_range, (idx64 // blk) // blocks_per_rank, idx64 % my_size)
            local = torch.where(in_range, idx64 - bucket * blk * blocks_per_rank, idx64 // my_size)
        else:
            in_range = idx64 < blk * my_size
            bucket = torch.where(in_range, idx64 // blk.clamp(min=1), idx64 % my_size)
            local = torch.where(in_range, idx64 - bucket * blk, idx64 // my_size)
    key = bucket * n_bags + bag_id
    new_lengths = torch.bincount(key, minlength=my_size * n_bags).to(lengths.dtype)
    order = torch.sort(key, stable=True).indices
    src_vals = idx64 if keep_orig_idx else local
    new_indices = src_vals.index_select(0, order).to(indices.dtype)
    new_weights = None if weights is None else weights.index_select(0, order)
    new_pos = None
    if bucketize_pos:
        starts = asynchronous_complete_cumsum(len64)[:-1]
        pos = torch.arange(N, device=dev) - starts.index_select(0, bag_id)
        new_pos = pos.index_select(0, order).to(indices.dtype)
    unbucketize = None
    if sequence:
        unbucketize = torch.empty(N, dtype=indices.dtype, device=dev)
        unbucketize[order] = torch.arange(N, device=dev, dtype=indices.dtype)
    return new_lengths, new_indices, new_weights, new_pos, unbucketize


# --------------------------------------------------------------------------------------
# jagged <-> dense
# --------------------------------------------------------------------------------------
class _JaggedToPadded(torch.autograd.Function):
    """The kernels are each other's adjoint: padding positions receive no gradient, truncated rows get zero."""

    @staticmethod
    def forward(ctx, values, offsets, max_length, padding_value):
        ctx.save_for_backward(offsets)
        ctx.total = values.shape[0]
        return torch.ops.trb200.jagged_to_padded_dense(values, offsets, max_length, padding_value)

    @staticmethod
    def backward(ctx, grad):
        (offsets,) = ctx.saved_tensors
        return torch.ops.trb200.padded_dense_to_jagged(grad.contiguous(), offsets, ctx.total), None, None, None


class _PaddedToJagged(torch.autograd.Function):
    @staticmethod
    def forward(ctx, dense, offsets, total):
        ctx.save_for_backward(offsets)
        ctx.max_length = dense.shape[1]
        return torch.ops.trb200.padded_dense_to_jagged(dense, offsets, total)

    @staticmethod
    def backward(ctx, grad):
        (offsets,) = ctx.saved_tensors
        return torch.ops.trb200.jagged_to_padded_dense(grad.contiguous(), offsets, ctx.max_length, 0.0), None, None


def jagged_to_padded_dense(
    values: torch.Tensor, offsets: torch.Tensor, max_length: int, padding_value: float = 0.0
) -> torch.Tensor:
    """``values [N(, D)]`` + ``offsets [B+1]`` -> ``[B, max_length(, D)]`` (truncating long bags)."""
    if values.is_cuda and values.numel() > 0 and values.dim() == 2 and _kern(values, "jagged_to_padded_dense"):
        if values.requires_grad and torch.is_grad_enabled():
            return _JaggedToPadded.apply(values, offsets, max_length, float(padding_value))
        return torch.ops.trb200.jagged_to_padded_dense(values, offsets, max_length, float(padding_value))
    B = offsets.numel() - 1
    off = offsets.to(torch.int64)
    lens = off[1:] - off[:-1]
    pos = torch.arange(max_length, device=values.device).view(1, -1)
    mask = pos < lens.view(-1, 1)
    src = (off[:-1].view(-1, 1) + pos).clamp(max=max(values.shape[0] - 1, 0))
    if values.shape[0] == 0:
        return values.new_full((B, max_length) + tuple(values.shape[1:]), padding_value)
    g = values.index_select(0, src.reshape(-1)).view((B, max_length) + tuple(values.shape[1:]))
    m = mask.view((B, max_length) + (1,) * (values.dim() - 1))
    return torch.where(m, g, torch.full_like(g, padding_value))


def padded_dense_to_jagged(dense: torch.Tensor, offsets: torch.Tensor, total: Optional[int] = None) -> torch.Tensor:
    """Inverse of :func:`jagged_to_padded_dense`: keep the first ``len[b]`` rows of every sample."""
    if dense.is_cuda and dense.dim() == 3 and dense.numel() > 0 and _kern(dense, "padded_dense_to_jagged"):
        if total is None:
            total = int(offsets[-1].item())
        if dense.requires_grad and torch.is_grad_enabled():
            return _PaddedToJagged.apply(dense, offsets, total)
        return torch.ops.trb200.padded_dense_to_jagged(dense, offsets, total)
    B, L = dense.shape[0], dense.shape[1]
    off = offsets.to(torch.int64)
    lens = (off[1:] - off[:-1]).clamp(max=L)
    pos = torch.arange(L, device=dense.device).view(1, -1)
    mask = pos < lens.view(-1, 1)
    return dense[mask]


def jagged_2d_to_dense(values: torch.Tensor, offsets: torch.Tensor, max_sequence_length: int) -> torch.Tensor:
    return jagged_to_padded_dense(values, offsets, max_sequence_length, 0.0)


def jagged_1d_to_dense(values: torch.Tensor, offsets: torch.Tensor, max_sequence_length: int, padding_value=0):
    return jagged_to_padded_dense(values, offsets, max_sequence_length, padding_value)


# --------------------------------------------------------------------------------------
# dedup
# --------------------------------------------------------------------------------------
_key_bits_cache: dict = {}


def _key_bits(feat_base: torch.Tensor, indices: torch.Tensor, bound: Optional[torch.Tensor]) -> int:
    """Bits the radix sort has to look at: enough for the largest linearized id.  ``bound`` (any tensor whose maximum is the total
    number of rows of all tables) gives it exactly; without it the ids' own width is bounded by their dtype.  The bases rarely
    change, so the one host read this needs is cached per tensor."""
    src = feat_base if bound is None else bound
    key = (src.data_ptr(), src.numel(), indices.dtype, bound is None)
    bits = _key_bits_cache.get(key)
    if bits is None:
        top = int(src.max().item()) if src.numel() else 0
        bits = top.bit_length() + 1 if bound is not None else min(64, max(top.bit_length(), 31 if indices.dtype == torch.int32 else 40) + 1)
        if len(_key_bits_cache) > 64:
            _key_bits_cache.clear()
        _key_bits_cache[key] = bits
    return bits


def unique_ids_per_feature(feat_base: torch.Tensor, offsets: torch.Tensor, indices: torch.Tensor,
                           bound: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``(distinct ids per feature [F], unique ids, reverse index)`` for ids in feature-major bags; ``feat_base [F]`` (ascending) is the
    id base of every feature's table: two features with the same base share a table and are deduplicated together (their ids
    are counted under the last of them).  Unique ids are feature-major and ascending inside a feature;
    ``unique[reverse[i]] == indices[i]``.  CUDA: sort-based kernels in ``sparse_small_kernels.cu``; elsewhere ``torch.unique``."""
    F = feat_base.numel()
    N = indices.numel()
    base = feat_base.to(torch.int64)
    if _kern(indices, "jagged_unique_indices") and N > 0:
        return torch.ops.trb200.jagged_unique_indices(base.contiguous(), offsets.to(torch.int64).contiguous(), indices.contiguous(), _key_bits(base, indices, bound))
    off = offsets.to(torch.int64)
    B = max((off.numel() - 1) // max(F, 1), 1)
    feat = lengths_range(off[1:] - off[:-1], N) // B if N else indices.to(torch.int64)
    lin = indices.to(torch.int64) + base.index_select(0, feat) if N else indices.to(torch.int64)
    uniq, reverse = torch.unique(lin, sorted=True, return_inverse=True)
    ufeat = torch.bucketize(uniq, base, right=True) - 1 if uniq.numel() else uniq
    counts = torch.bincount(ufeat, minlength=F) if uniq.numel() else torch.zeros(F, dtype=torch.int64, device=indices.device)
    unique = (uniq - base.index_select(0, ufeat)) if uniq.numel() else uniq
    return counts, unique.to(indices.dtype), reverse.to(indices.dtype)


def jagged_unique_indices(
    hash_size_cumsum: torch.Tensor,
    hash_size_offsets: torch.Tensor,
    offsets: torch.Tensor,
    indices: torch.Tensor,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Per-feature deduplication of ids.

    ``offsets [F*B+1]`` describe the bags, ``hash_size_cumsum`` gives every table's id base
    and ``hash_size_offsets [F+1]`` maps features to tables.  Returns
    ``(output_lengths [F], output_offsets [F+1], unique_indices, reverse_index)`` where
    ``unique_indices[output_offsets[f]:output_offsets[f+1]]`` are the sorted distinct ids of
    feature ``f`` and ``unique_indices[reverse_index[i]] == indices[i]``.
    """
    base = hash_size_cumsum.to(torch.int64)[hash_size_offsets.to(torch.int64)[:-1]]
    out_len, unique_indices, reverse = unique_ids_per_feature(base, offsets, indices, bound=hash_size_cumsum)
    out_off = asynchronous_complete_cumsum(out_len)
    return out_len.to(offsets.dtype), out_off.to(offsets.dtype), unique_indices, reverse


# --------------------------------------------------------------------------------------
# pooled-embedding column permutes
# --------------------------------------------------------------------------------------
def permute_pooled_embs(pooled: torch.Tensor, dims: List[int], permute: List[int]) -> torch.Tensor:
    """Reorder the column blocks (widths ``dims``) of ``pooled [B, sum(dims)]`` by ``permute``."""
    offs = [0]
    for d in dims:
        offs.append(offs[-1] + d)
    cols = torch.cat(
        [torch.arange(offs[p], offs[p + 1], device=pooled.device) for p in permute]
    ) if permute else torch.empty(0, dtype=torch.int64, device=pooled.device)
    return pooled.index_select(1, cols)


class RegroupPlan:
    """Descriptor tables of one regroup (which column block of which input feeds which block of which group) for the one-launch
    kernel, forward and backward, kept on the device."""

    def __init__(self, in_lengths: List[List[int]], in_keys: List[List[str]], groups: List[List[str]], device: torch.device) -> None:
        loc = {}
        for ti, (keys, lens) in enumerate(zip(in_keys, in_lengths)):
            o = 0
            for k, l in zip(keys, lens):
                if k not in loc:
                    loc[k] = (ti, o, l)
                o += l
        self.in_widths = [sum(l) for l in in_lengths]
        self.out_widths = [sum(loc[k][2] for k in g) for g in groups]
        fwd_desc, fwd_src = [], []
        readers = {}  # (in tensor, in offset, len) -> [(group, offset in group)]
        for gi, g in enumerate(groups):
            o = 0
            for k in g:
                ti, io, l = loc[k]
                fwd_desc.append([gi, o, l, len(fwd_src), 1])
                fwd_src.append([ti, io])
                readers.setdefault((ti, io, l), []).append((gi, o))
                o += l
        bwd_desc, bwd_src = [], []
        for ti, (keys, lens) in enumerate(zip(in_keys, in_lengths)):
            o = 0
            for k, l in zip(keys, lens):
                rs = readers.get((ti, o, l), []) if loc[k] == (ti, o, l) else []
                bwd_desc.append([ti, o, l, len(bwd_src), len(rs)])
                bwd_src.extend([list(r) for r in rs])
                o += l
        mk = lambda rows, w: torch.tensor(rows if rows else [[0] * w][:0], dtype=torch.int32, device=device).reshape(-1, w)
        self.fwd_desc, self.fwd_src = mk(fwd_desc, 5), mk(fwd_src, 2)
        self.bwd_desc, self.bwd_src = mk(bwd_desc, 5), mk(bwd_src, 2)


class _KTRegroup(torch.autograd.Function):
    @staticmethod
    def forward(ctx, plan: RegroupPlan, *values: torch.Tensor):
        ctx.plan = plan
        outs = torch.ops.trb200.kt_regroup([v if v.stride(1) == 1 else v.contiguous() for v in values], plan.out_widths, plan.fwd_desc, plan.fwd_src)
        return tuple(outs)

    @staticmethod
    def backward(ctx, *grads: torch.Tensor):
        plan = ctx.plan
        B = next(g.shape[0] for g in grads if g is not None)
        ref = next(g for g in grads if g is not None)
        gs = [g if g is not None else ref.new_zeros(B, w) for g, w in zip(grads, plan.out_widths)]
        gs = [g if g.stride(1) == 1 else g.contiguous() for g in gs]
        return (None, *torch.ops.trb200.kt_regroup(gs, plan.in_widths, plan.bwd_desc, plan.bwd_src))


_REGROUP_PLANS = {}


def permute_multi_embedding(
    values: List[torch.Tensor], in_lengths: List[List[int]], in_keys: List[List[str]], groups: List[List[str]]
) -> List[torch.Tensor]:
    """Gather key-blocks from several ``[B, sum(D)]`` tensors into grouped outputs.

    Differentiable; a key may appear in several groups (its gradients are summed).  On a CUDA device the whole regroup is one
    kernel launch forward and one backward (``kt_regroup``); elsewhere it is built from ``narrow``/``cat``.
    """
    v0 = values[0]
    if v0.is_cuda and len(values) <= 32 and len(groups) <= 32 and all(v.dtype == v0.dtype and v.dim() == 2 for v in values) and _kern(v0, "kt_regroup"):
        key = (tuple(tuple(l) for l in in_lengths), tuple(tuple(k) for k in in_keys), tuple(tuple(g) for g in groups), v0.device)
        plan = _REGROUP_PLANS.get(key)
        if plan is None:
            plan = _REGROUP_PLANS[key] = RegroupPlan(in_lengths, in_keys, groups, v0.device)
        return list(_KTRegroup.apply(plan, *values))
    loc = {}
    for ti, (keys, lens) in enumerate(zip(in_keys, in_lengths)):
        o = 0
        for k, l in zip(keys, lens):
            if k not in loc:
                loc[k] = (ti, o, l)
            o += l
    outs = []
    for g in groups:
        parts = [values[loc[k][0]].narrow(1, loc[k][1], loc[k][2]) for k in g]
        outs.append(torch.cat(parts, dim=1) if len(parts) > 1 else parts[0].contiguous())
    return outs


# --------------------------------------------------------------------------------------
# managed-collision hash and pruning remap
# --------------------------------------------------------------------------------------
ZCH_NO_EVICT, ZCH_TTL, ZCH_LRU = 0, 1, 2
ZCH_EMPTY_SCORE = 2**31 - 1


def zch_probe(
    ids: torch.Tensor,
    identities: torch.Tensor,
    metadata: Optional[torch.Tensor],
    segments: torch.Tensor,
    input_hash_size: int = 0,
    out_offset: int = 0,
    max_probe: int = 128,
    readonly: bool = False,
    disable_fallback: bool = False,
    input_metadata: Optional[torch.Tensor] = None,
    eviction_threshold: int = -1,
    eviction_policy: int = ZCH_NO_EVICT,
    reserved_slots: int = 0,
    admit: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Multi-probe zero-collision hash: ``ids -> (slot, evicted_slot)`` against the slot table ``identities`` (-1 = empty),
    updated in place unless ``readonly``.  ``segments`` are the global boundaries of the hash buckets, the table covers the slots
    ``[out_offset, out_offset + len(identities))``.  A miss claims an empty slot among the ``max_probe`` slots after its hash
    position inside its bucket, or evicts one whose score in ``metadata`` expired (TTL) / is the oldest (LRU); with no slot free it
    shares the row at its hash position, or gets -1 with ``disable_fallback``.  Duplicate ids are resolved once.
    Opt-in admission: with ``reserved_slots > 0`` the last ``reserved_slots`` slots of every bucket are never claimed; an id without a slot
    of its own shares one of them (by hash).  ``admit`` (bool per id) says which ids may claim a slot in this call: the others are
    only looked up (an id occurring several times is admitted if any occurrence is).
    CUDA: ``misc_kernels.cu`` (lookup and insert launches); CPU: ``csrc/cpu/sparse_cpu.cpp``."""
    ids = ids.to(torch.int64).contiguous()
    if admit is not None and not readonly and ids.numel() > 0:
        admit = admit.to(device=ids.device, dtype=torch.bool)
        if bool(admit.all()):
            admit = None
    if admit is not None and not readonly and ids.numel() > 0:
        # an id with several occurrences must take one path: admitted if any occurrence drew admission
        uniq, inverse = torch.unique(ids, return_inverse=True)
        any_admit = torch.zeros(uniq.numel(), dtype=torch.int32, device=ids.device).scatter_reduce_(0, inverse, admit.to(torch.int32), reduce="amax", include_self=True)
        admit = any_admit.index_select(0, inverse).bool()
        slots, evicted = torch.empty_like(ids), torch.full_like(ids, -1)
        common = dict(input_hash_size=input_hash_size, out_offset=out_offset, max_probe=max_probe, disable_fallback=disable_fallback,
                      eviction_threshold=eviction_threshold, eviction_policy=eviction_policy, reserved_slots=reserved_slots)
        meta_of = (lambda m: None) if input_metadata is None else (lambda m: input_metadata[m])
        if bool(admit.any()):
            slots[admit], evicted[admit] = zch_probe(ids[admit], identities, metadata, segments, readonly=False, input_metadata=meta_of(admit), **common)
        rest = ~admit
        slots[rest], _ = zch_probe(ids[rest], identities, metadata, segments, readonly=True, input_metadata=meta_of(rest), **common)
        return slots, evicted
    args = (identities, metadata, segments.to(device=ids.device, dtype=torch.int64), int(input_hash_size), int(out_offset), int(max_probe), bool(readonly),
            bool(disable_fallback), None if input_metadata is None else input_metadata.to(torch.int32).contiguous(), int(eviction_threshold), int(eviction_policy),
            int(reserved_slots))
    op = torch.ops.trb200.zch_probe if _kern(ids, "zch_probe") else _ext.cpu_ops().zch_probe
    if readonly or ids.numel() == 0:
        return op(ids, *args)
    # one probe per distinct id: two copies of a new id must not race for two slots
    uniq, inverse = torch.unique(ids, return_inverse=True)
    um = None
    if args[8] is not None:
        um = torch.zeros(uniq.numel(), dtype=torch.int32, device=ids.device).scatter_reduce_(0, inverse, args[8], reduce="amax", include_self=False)
    slots, evicted = op(uniq, *args[:8], um, *args[9:])
    ev = torch.full_like(ids, -1)
    first = torch.full((uniq.numel(),), ids.numel(), dtype=torch.int64, device=ids.device).scatter_reduce_(
        0, inverse, torch.arange(ids.numel(), device=ids.device), reduce="amin", include_self=True)
    ev[first] = evicted
    return slots.index_select(0, inverse), ev


def itep_remap(values: torch.Tensor, feature_offsets: torch.Tensor, feature_buffer: torch.Tensor, address_lookup: torch.Tensor, row_util: torch.Tensor,
               buffer_offsets: torch.Tensor, update_util: bool) -> torch.Tensor:
    """Remap the ids of pruned tables through ``address_lookup`` (entry ``v >= 0``: own row ``v``; ``v < 0``: shared row
    ``-(v+1)``) and, when ``update_util``, add one to ``row_util`` of every id seen.  ``feature_offsets [F+1]`` cuts ``values`` into
    features, ``feature_buffer [F]`` (int32) names each feature's buffer or -1."""
    v = values.to(torch.int64).contiguous()
    op = torch.ops.trb200.itep_remap if _kern(v, "itep_remap") else _ext.cpu_ops().itep_remap
    return op(v, feature_offsets.to(device=v.device, dtype=torch.int64), feature_buffer.to(device=v.device, dtype=torch.int32), address_lookup, row_util,
              buffer_offsets.to(device=v.device, dtype=torch.int64), bool(update_util)).to(values.dtype)


# --------------------------------------------------------------------------------------
# variable batch per feature: expand deduplicated pooled rows to the full batch
# --------------------------------------------------------------------------------------
class _VbeExpand(torch.autograd.Function):
    @staticmethod
    def forward(ctx, flat, inverse, rows_per_feature, dims):
        desc, base, col = [], 0, 0
        for b, d in zip(rows_per_feature, dims):
            desc.append([base, b, d, col])
            base += b * d
            col += d
        err = torch.zeros(1, dtype=torch.int32, device=flat.device)
        out = torch.ops.trb200.vbe_expand(flat.contiguous(), torch.tensor(desc, dtype=torch.int64).to(flat.device, non_blocking=True),
                                          inverse.contiguous(), col, err)
        ctx.save_for_backward(inverse)
        ctx.layout = (desc, flat.numel())
        return out

    @staticmethod
    def backward(ctx, grad):
        (inverse,) = ctx.saved_tensors
        desc, n = ctx.layout
        g = grad.new_zeros(n)
        for f, (base, b, d, col) in enumerate(desc):  # rows that several samples share collect all their gradients
            g[base: base + b * d].view(b, d).index_add_(0, inverse[f].to(torch.int64), grad[:, col: col + d])
        return g, None, None, None


def vbe_expand(flat: torch.Tensor, inverse: torch.Tensor, rows_per_feature: List[int], dims: List[int]) -> torch.Tensor:
    """``flat`` holds, feature after feature, the pooled rows ``[rows_f, dim_f]`` of the deduplicated batches; ``inverse [F, B]``
    names for every sample of the full batch the row to use.  Returns ``[B, sum(dim_f)]``."""
    if flat.is_cuda and inverse.dtype in (torch.int32, torch.int64) and _kern(flat, "vbe_expand"):
        return _VbeExpand.apply(flat, inverse, list(rows_per_feature), list(dims))
    outs, base = [], 0
    for f, (b, d) in enumerate(zip(rows_per_feature, dims)):
        outs.append(flat[base: base + b * d].view(b, d).index_select(0, inverse[f].to(torch.int64)))
        base += b * d
    return torch.cat(outs, dim=1)
