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
def jagged_to_padded_dense(
    values: torch.Tensor, offsets: torch.Tensor, max_length: int, padding_value: float = 0.0
) -> torch.Tensor:
    """``values [N(, D)]`` + ``offsets [B+1]`` -> ``[B, max_length(, D)]`` (truncating long bags)."""
    if values.is_cuda and values.numel() > 0 and values.dim() == 2 and _kern(values, "jagged_to_padded_dense"):
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
    F = hash_size_offsets.numel() - 1
    n_bags = offsets.numel() - 1
    B = n_bags // max(F, 1)
    off = offsets.to(torch.int64)
    N = indices.numel()
    bag = lengths_range(off[1:] - off[:-1], N)
    feat = bag // max(B, 1)
    base = hash_size_cumsum.to(torch.int64)[hash_size_offsets.to(torch.int64)[:-1]]
    lin = indices.to(torch.int64) + base.index_select(0, feat) if N else indices.to(torch.int64)
    uniq, reverse = torch.unique(lin, sorted=True, return_inverse=True)
    ufeat = torch.bucketize(uniq, base, right=True) - 1 if uniq.numel() else uniq
    out_len = torch.bincount(ufeat, minlength=F) if uniq.numel() else torch.zeros(F, dtype=torch.int64, device=indices.device)
    out_off = asynchronous_complete_cumsum(out_len)
    unique_indices = (uniq - base.index_select(0, ufeat)) if uniq.numel() else uniq
    return out_len.to(offsets.dtype), out_off.to(offsets.dtype), unique_indices.to(indices.dtype), reverse.to(indices.dtype)


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


def permute_multi_embedding(
    values: List[torch.Tensor], in_lengths: List[List[int]], in_keys: List[List[str]], groups: List[List[str]]
) -> List[torch.Tensor]:
    """Gather key-blocks from several ``[B, sum(D)]`` tensors into grouped outputs.

    Differentiable (built from ``narrow``/``cat``); duplicates across groups are allowed
    and their gradients are summed by autograd.
    """
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
