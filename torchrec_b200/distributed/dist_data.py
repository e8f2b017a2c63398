"""Distribution modules for sparse inputs and embedding outputs (NCCL / gloo path).

* ``KJTAllToAll``: two-stage redistribution of a ``KeyedJaggedTensor`` -- a small integer
  all-to-all of split sizes (needed to size receive buffers; costs one device-to-host read), then
  one all-to-all per payload tensor (lengths, values, optional strides/weights), then the recat
  permute into key-major order.
* ``PooledEmbeddingsAllToAll`` / ``PooledEmbeddingsReduceScatter`` / ``PooledEmbeddingsAllGather`` /
  ``SequenceEmbeddingsAllToAll``: module wrappers around the autograd collectives of ``comm_ops``.
* ``KJTOneToAll`` / ``EmbeddingsAllToOne`` ...: single-process multi-device copies for inference.

Counterpart of ``torchrec/distributed/dist_data.py`` (splits ``:220-291``, tensors ``:294-442``,
``KJTAllToAll`` ``:583``, pooled a2a ``:897``, reduce-scatter ``:1250``, sequence a2a ``:1493``).
"""
from __future__ import annotations

import itertools
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import nn
from torch.autograd.profiler import record_function

from torchrec_b200.distributed.comm_ops import (
    all_gather_base_pooled,
    alltoall_pooled,
    alltoall_sequence,
    reduce_scatter_base_pooled,
    reduce_scatter_v_pooled,
    variable_batch_alltoall_pooled,
)
from torchrec_b200.distributed.types import Awaitable, NoWait, QuantizedCommCodecs
from torchrec_b200.ops import sparse_ops as sops
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


def _get_recat(
    local_split: int,
    num_splits: int,
    stagger: int = 1,
    device: Optional[torch.device] = None,
    batch_size_per_rank: Optional[List[int]] = None,
) -> Optional[torch.Tensor]:
    """Permutation that turns (source rank, key)-major received data into key-major order.

    ``_get_recat(2, 4, 1) -> [0, 2, 4, 6, 1, 3, 5, 7]``; ``stagger`` interleaves source ranks for
    the hierarchical (TWRW) layout: ``_get_recat(2, 4, 2) -> [0, 4, 2, 6, 1, 5, 3, 7]``.
    With different batch sizes per rank the segment permutation is expanded to a per-bag permutation.
    """
    if local_split == 0:
        return None
    vb_key = tuple(batch_size_per_rank) if batch_size_per_rank is not None and any(bs != batch_size_per_rank[0] for bs in batch_size_per_rank) else None
    cache_key = (local_split, num_splits, stagger, str(device), vb_key)
    cached = _RECAT_CACHE.get(cache_key)
    if cached is not None:
        return cached
    out = _build_recat(local_split, num_splits, stagger, device, batch_size_per_rank)
    if len(_RECAT_CACHE) >= 256:
        _RECAT_CACHE.clear()
    _RECAT_CACHE[cache_key] = out
    return out


# Building the permutation on the device is a host-to-device copy from pageable memory, which stalls the host until the stream
# has drained; the permutation only depends on the layout of the exchange, so it is built once per layout.
_RECAT_CACHE: Dict[Tuple[Any, ...], torch.Tensor] = {}


def _build_recat(local_split: int, num_splits: int, stagger: int, device: Optional[torch.device], batch_size_per_rank: Optional[List[int]]) -> torch.Tensor:
    feature_order = [x + num_splits // stagger * y for x in range(num_splits // stagger) for y in range(stagger)]
    recat = [i + j * local_split for i in range(local_split) for j in feature_order]
    vb = batch_size_per_rank is not None and any(bs != batch_size_per_rank[0] for bs in batch_size_per_rank)
    if vb:
        batch_size_per_feature = list(itertools.chain.from_iterable(itertools.repeat(x, local_split) for x in batch_size_per_rank))
        permuted = [batch_size_per_feature[r] for r in recat]
        input_offset = [0] + list(itertools.accumulate(batch_size_per_feature))
        output_offset = [0] + list(itertools.accumulate(permuted))
        return sops.expand_into_jagged_permute(
            torch.tensor(recat, device=device, dtype=torch.int32),
            torch.tensor(input_offset, device=device, dtype=torch.int32),
            torch.tensor(output_offset, device=device, dtype=torch.int32),
            output_offset[-1],
        )
    return torch.tensor(recat, device=device, dtype=torch.int32)


class SplitsAllToAllAwaitable(Awaitable[List[List[int]]]):
    """All-to-all of the per-destination split sizes; ``wait()`` returns them as Python lists."""

    def __init__(self, input_tensors, pg: dist.ProcessGroup, device: Optional[torch.device] = None) -> None:
        """``input_tensors``: one ``[world]`` tensor per quantity, or (cheaper) one Python list per quantity together with ``device``:
        the lists are interleaved on the host and cross to the device in a single copy."""
        super().__init__()
        self.num_workers: int = pg.size()
        with record_function("## all2all_data:kjt splits ##"):
            if len(input_tensors) > 0 and not isinstance(input_tensors[0], torch.Tensor):
                flat = [int(s[w]) for w in range(self.num_workers) for s in input_tensors]
                input_tensor = torch.tensor(flat, dtype=torch.int64, device=device)
                self._output_tensor = torch.empty_like(input_tensor)
            else:
                self._output_tensor = torch.empty(
                    [self.num_workers * len(input_tensors)], device=input_tensors[0].device, dtype=input_tensors[0].dtype
                )
                input_tensor = torch.stack(input_tensors, dim=1).flatten()
            self._splits_awaitable = dist.all_to_all_single(output=self._output_tensor, input=input_tensor, group=pg, async_op=True)

    def _wait_impl(self) -> List[List[int]]:
        self._splits_awaitable.wait()
        return self._output_tensor.view(self.num_workers, -1).T.tolist()


class KJTAllToAllTensorsAwaitable(Awaitable[KeyedJaggedTensor]):
    """Second stage of the KJT redistribution: payload all-to-alls, then ``KeyedJaggedTensor.dist_init``."""

    def __init__(
        self,
        pg: dist.ProcessGroup,
        input: KeyedJaggedTensor,
        splits: List[int],
        input_splits: List[List[int]],
        output_splits: List[List[int]],
        input_tensors: List[torch.Tensor],
        labels: List[str],
        keys: List[str],
        device: torch.device,
        stagger: int,
        stride_per_rank: Optional[List[int]],
    ) -> None:
        super().__init__()
        self._workers = pg.size()
        self._pg = pg
        self._device = device
        self._input = input
        self._splits = splits
        self._input_splits: Dict[str, List[int]] = dict(zip(labels, input_splits))
        self._output_splits: Dict[str, List[int]] = dict(zip(labels, output_splits))
        self._keys = keys
        self._stagger = stagger
        self._stride_per_rank = stride_per_rank
        self._recat: Optional[torch.Tensor] = _get_recat(
            local_split=splits[pg.rank()], num_splits=len(splits), stagger=stagger, device=device,
            batch_size_per_rank=self._stride_per_rank,
        )
        if self._workers == 1:
            return
        self._output_tensors: List[torch.Tensor] = []
        self._awaitables = []
        for input_split, output_split, input_tensor, label in zip(input_splits, output_splits, input_tensors, labels):
            output_tensor = torch.empty(sum(output_split), device=self._device, dtype=input_tensor.dtype)
            with record_function(f"## all2all_data:kjt {label} ##"):
                awaitable = dist.all_to_all_single(
                    output=output_tensor, input=input_tensor.contiguous(), output_split_sizes=output_split,
                    input_split_sizes=input_split, group=self._pg, async_op=True,
                )
            self._output_tensors.append(output_tensor)
            self._awaitables.append(awaitable)

    def _wait_impl(self) -> KeyedJaggedTensor:
        if self._workers == 1:
            self._input.sync()
            return self._input
        for a in self._awaitables:
            a.wait()
        return type(self._input).dist_init(
            keys=self._keys,
            tensors=self._output_tensors,
            variable_stride_per_key=self._input.variable_stride_per_key(),
            num_workers=self._workers,
            recat=self._recat,
            stride_per_rank=self._stride_per_rank,
            stagger=self._stagger,
        )


class KJTAllToAllSplitsAwaitable(Awaitable[KJTAllToAllTensorsAwaitable]):
    """First stage: exchange split sizes so that every rank can size its receive buffers."""

    def __init__(self, pg: dist.ProcessGroup, input: KeyedJaggedTensor, splits: List[int], labels: List[str],
                 tensor_splits: List[List[int]], input_tensors: List[torch.Tensor], keys: List[str], device: torch.device, stagger: int,
                 defer_splits_exchange: bool = False) -> None:
        super().__init__()
        self._workers = pg.size()
        self._pg = pg
        self._device = device
        self._input = input
        self._splits = splits
        self._labels = labels
        self._input_splits = tensor_splits
        self._input_tensors = input_tensors
        self._keys = keys
        self._stagger = stagger
        self._output_splits: List[List[int]] = self._input_splits
        self._stride_per_rank: Optional[List[int]] = None if self._input.variable_stride_per_key() else [self._input.stride()] * self._workers
        self._splits_awaitable: Optional[SplitsAllToAllAwaitable] = None
        # a train pipeline exchanges the split sizes of all its modules in one fused collective instead
        if self._workers == 1 or defer_splits_exchange:
            return
        self._launch_splits_exchange()

    def _launch_splits_exchange(self) -> None:
        lists = [list(s) for s in self._input_splits]
        if not self._input.variable_stride_per_key():
            lists.append([self._input.stride()] * self._workers)
        self._splits_awaitable = SplitsAllToAllAwaitable(lists, self._pg, device=self._device)

    def _wait_impl(self) -> KJTAllToAllTensorsAwaitable:
        if self._workers > 1:
            if self._splits_awaitable is None:
                self._launch_splits_exchange()
            output_list = self._splits_awaitable.wait()
            if self._input.variable_stride_per_key():
                self._output_splits = output_list
            else:
                self._output_splits = output_list[:-1]
                self._stride_per_rank = output_list[-1]
        return KJTAllToAllTensorsAwaitable(
            pg=self._pg, input=self._input, splits=self._splits, input_splits=self._input_splits,
            output_splits=self._output_splits, input_tensors=self._input_tensors, labels=self._labels,
            keys=self._keys, device=self._device, stagger=self._stagger, stride_per_rank=self._stride_per_rank,
        )


class KJTAllToAll(nn.Module):
    """Send keys ``[sum(splits[:r]), sum(splits[:r+1]))`` of every rank's KJT to rank ``r``.

    The result on rank ``r`` has ``splits[r]`` keys and the concatenated batch of all ranks.
    """

    def __init__(self, pg: dist.ProcessGroup, splits: List[int], stagger: int = 1) -> None:
        super().__init__()
        assert len(splits) == pg.size(), "splits must have one entry per rank"
        self._pg = pg
        self._splits = splits
        self._splits_cumsum = [0] + list(itertools.accumulate(splits))
        self._stagger = stagger
        self.defer_splits_exchange: bool = False  # set by train pipelines that fuse the split exchange

    def forward(self, input: KeyedJaggedTensor) -> Awaitable[KJTAllToAllTensorsAwaitable]:
        with torch.no_grad():
            assert len(input.keys()) == sum(self._splits)
            rank = dist.get_rank(self._pg)
            local_keys = input.keys()[self._splits_cumsum[rank]: self._splits_cumsum[rank + 1]]
            return KJTAllToAllSplitsAwaitable(
                pg=self._pg, input=input, splits=self._splits, labels=input.dist_labels(),
                tensor_splits=input.dist_splits(self._splits), input_tensors=input.dist_tensors(),
                keys=local_keys, device=input.device(), stagger=self._stagger,
                defer_splits_exchange=self.defer_splits_exchange,
            )


class KJTOneToAll(nn.Module):
    """Split a KJT by keys and copy piece ``r`` to device ``r`` (one process, many devices)."""

    def __init__(self, splits: List[int], world_size: int, device: Optional[torch.device] = None) -> None:
        super().__init__()
        self._splits = splits
        self._world_size = world_size
        self._device_type = "meta" if device is not None and device.type == "meta" else ("cuda" if torch.cuda.is_available() else "cpu")
        assert self._world_size == len(splits)

    def forward(self, kjt: KeyedJaggedTensor):
        from torchrec_b200.distributed.embedding_types import KJTList

        kjts = kjt.split(self._splits)
        out = []
        for rank in range(self._world_size):
            dev = torch.device(self._device_type, rank) if self._device_type == "cuda" else torch.device(self._device_type)
            out.append(kjts[rank].to(dev, non_blocking=True))
        return NoWait(KJTList(out))


# ---- pooled outputs ------------------------------------------------------------------------------
class PooledEmbeddingsAwaitable(Awaitable[torch.Tensor]):
    def __init__(self, tensor_awaitable: Awaitable[torch.Tensor]) -> None:
        super().__init__()
        self._tensor_awaitable = tensor_awaitable

    def _wait_impl(self) -> torch.Tensor:
        return self._tensor_awaitable.wait()

    @property
    def callbacks(self) -> List[Callable[[torch.Tensor], torch.Tensor]]:
        return self._callbacks


class PooledEmbeddingsAllToAll(nn.Module):
    """``[B_global, D_local_sum]`` -> ``[B_local, sum_r D_r]`` (table-wise / column-wise output dist)."""

    def __init__(self, pg: dist.ProcessGroup, dim_sum_per_rank: List[int], device: Optional[torch.device] = None,
                 callbacks: Optional[List[Callable[[torch.Tensor], torch.Tensor]]] = None,
                 codecs: Optional[QuantizedCommCodecs] = None) -> None:
        super().__init__()
        self._pg = pg
        self._callbacks = callbacks or []
        self._dim_sum_per_rank = dim_sum_per_rank
        self._codecs = codecs
        self.register_buffer("_dim_sum_per_rank_tensor", torch.tensor(dim_sum_per_rank, device=device, dtype=torch.int), persistent=False)
        cumsum = list(itertools.accumulate(dim_sum_per_rank))
        self.register_buffer("_cumsum_dim_sum_per_rank_tensor", torch.tensor(cumsum, device=device, dtype=torch.int), persistent=False)

    def forward(self, local_embs: torch.Tensor, batch_size_per_rank: Optional[List[int]] = None) -> PooledEmbeddingsAwaitable:
        if local_embs.numel() == 0:
            local_embs.view(local_embs.size(0) * self._pg.size(), 0)
        if batch_size_per_rank is None:
            B_global = local_embs.size(0)
            assert B_global % self._pg.size() == 0, f"num of ranks {self._pg.size()} doesn't divide global batch size {B_global}"
            batch_size_per_rank = [B_global // self._pg.size()] * self._pg.size()
        tensor_awaitable = alltoall_pooled(
            a2a_pooled_embs_tensor=local_embs, batch_size_per_rank=batch_size_per_rank,
            dim_sum_per_rank=self._dim_sum_per_rank, dim_sum_per_rank_tensor=self._dim_sum_per_rank_tensor,
            cumsum_dim_sum_per_rank_tensor=self._cumsum_dim_sum_per_rank_tensor, group=self._pg, codecs=self._codecs,
        )
        aw = PooledEmbeddingsAwaitable(tensor_awaitable)
        aw.callbacks.extend(self._callbacks)
        return aw

    @property
    def callbacks(self) -> List[Callable[[torch.Tensor], torch.Tensor]]:
        return self._callbacks


class VariableBatchPooledEmbeddingsAllToAll(nn.Module):
    """Pooled all-to-all when every (rank, feature) has its own batch size; payload is 1-D."""

    def __init__(self, pg: dist.ProcessGroup, emb_dim_per_rank_per_feature: List[List[int]], device: Optional[torch.device] = None,
                 callbacks: Optional[List[Callable[[torch.Tensor], torch.Tensor]]] = None, codecs: Optional[QuantizedCommCodecs] = None) -> None:
        super().__init__()
        self._pg = pg
        self._emb_dim_per_rank_per_feature = emb_dim_per_rank_per_feature
        self._callbacks = callbacks or []
        self._codecs = codecs

    def forward(self, local_embs: torch.Tensor, batch_size_per_rank_per_feature: List[List[int]], batch_size_per_feature_pre_a2a: List[int]) -> PooledEmbeddingsAwaitable:
        tensor_awaitable = variable_batch_alltoall_pooled(
            a2a_pooled_embs_tensor=local_embs, batch_size_per_rank_per_feature=batch_size_per_rank_per_feature,
            batch_size_per_feature_pre_a2a=batch_size_per_feature_pre_a2a,
            emb_dim_per_rank_per_feature=self._emb_dim_per_rank_per_feature, group=self._pg, codecs=self._codecs,
        )
        aw = PooledEmbeddingsAwaitable(tensor_awaitable)
        aw.callbacks.extend(self._callbacks)
        return aw

    @property
    def callbacks(self):
        return self._callbacks


class PooledEmbeddingsReduceScatter(nn.Module):
    """``[W*B, D]`` partial sums -> ``[B, D]`` (row-wise output dist); ``input_splits`` for uneven batches."""

    def __init__(self, pg: dist.ProcessGroup, codecs: Optional[QuantizedCommCodecs] = None) -> None:
        super().__init__()
        self._pg = pg
        self._codecs = codecs

    def forward(self, local_embs: torch.Tensor, input_splits: Optional[List[int]] = None) -> PooledEmbeddingsAwaitable:
        if input_splits and len(set(input_splits)) > 1:
            aw = reduce_scatter_v_pooled(local_embs, input_splits, self._pg, codecs=self._codecs)
        else:
            aw = reduce_scatter_base_pooled(local_embs, self._pg, codecs=self._codecs)
        return PooledEmbeddingsAwaitable(aw)


class VariableBatchPooledEmbeddingsReduceScatter(nn.Module):
    """Reduce-scatter of a flat per-feature variable-batch payload."""

    def __init__(self, pg: dist.ProcessGroup, codecs: Optional[QuantizedCommCodecs] = None) -> None:
        super().__init__()
        self._pg = pg
        self._codecs = codecs

    def forward(self, local_embs: torch.Tensor, batch_size_per_rank_per_feature: List[List[int]], embedding_dims: List[int]) -> PooledEmbeddingsAwaitable:
        splits = [sum(b * d for b, d in zip(bs, embedding_dims)) for bs in batch_size_per_rank_per_feature]
        return PooledEmbeddingsAwaitable(reduce_scatter_v_pooled(local_embs.view(-1), splits, self._pg, codecs=self._codecs))


class PooledEmbeddingsAllGather(nn.Module):
    def __init__(self, pg: dist.ProcessGroup, codecs: Optional[QuantizedCommCodecs] = None) -> None:
        super().__init__()
        self._pg = pg
        self._codecs = codecs

    def forward(self, local_emb: torch.Tensor) -> PooledEmbeddingsAwaitable:
        return PooledEmbeddingsAwaitable(all_gather_base_pooled(local_emb, self._pg, codecs=self._codecs))


# ---- sequence outputs ------------------------------------------------------------------------------
class SequenceEmbeddingsAwaitable(Awaitable[torch.Tensor]):
    def __init__(self, tensor_awaitable: Awaitable[torch.Tensor], unbucketize_permute_tensor: Optional[torch.Tensor], embedding_dim: int) -> None:
        super().__init__()
        self._tensor_awaitable = tensor_awaitable
        if unbucketize_permute_tensor is not None:
            self.callbacks.append(lambda ret: torch.index_select(ret.view(-1, embedding_dim), 0, unbucketize_permute_tensor.to(torch.int64)))

    def _wait_impl(self) -> torch.Tensor:
        return self._tensor_awaitable.wait()


class SequenceEmbeddingsAllToAll(nn.Module):
    """Return every looked-up row to the rank (and position) that requested it."""

    def __init__(self, pg: dist.ProcessGroup, features_per_rank: List[int], device: Optional[torch.device] = None,
                 codecs: Optional[QuantizedCommCodecs] = None) -> None:
        super().__init__()
        self._pg = pg
        self._local_split = features_per_rank[self._pg.rank()]
        self._num_splits = self._pg.size()
        # forward: (feature, source rank) -> (source rank, feature); backward: the inverse
        fwd = []
        for r in range(self._num_splits):
            for f in range(self._local_split):
                fwd.append(f * self._num_splits + r)
        bwd = [0] * len(fwd)
        for i, v in enumerate(fwd):
            bwd[v] = i
        self.register_buffer("_forward_recat_tensor", torch.tensor(fwd, device=device, dtype=torch.int), persistent=False)
        self.register_buffer("_backward_recat_tensor", torch.tensor(bwd, device=device, dtype=torch.int), persistent=False)
        self._codecs = codecs

    def forward(
        self,
        local_embs: torch.Tensor,
        lengths: torch.Tensor,
        input_splits: List[int],
        output_splits: List[int],
        unbucketize_permute_tensor: Optional[torch.Tensor] = None,
        batch_size_per_rank: Optional[List[int]] = None,
        sparse_features_recat: Optional[torch.Tensor] = None,
    ) -> SequenceEmbeddingsAwaitable:
        variable_batch_size = batch_size_per_rank is not None and len(set(batch_size_per_rank)) > 1
        if sparse_features_recat is not None:
            forward_recat_tensor = torch.empty_like(sparse_features_recat)
            forward_recat_tensor[sparse_features_recat.to(torch.int64)] = torch.arange(
                sparse_features_recat.numel(), device=sparse_features_recat.device, dtype=sparse_features_recat.dtype
            )
            backward_recat_tensor = sparse_features_recat
        else:
            forward_recat_tensor = self._forward_recat_tensor
            backward_recat_tensor = self._backward_recat_tensor
        tensor_awaitable = alltoall_sequence(
            a2a_sequence_embs_tensor=local_embs,
            forward_recat_tensor=forward_recat_tensor if self._local_split > 0 else None,
            backward_recat_tensor=backward_recat_tensor,
            lengths_after_sparse_data_all2all=lengths,
            input_splits=input_splits,
            output_splits=output_splits,
            variable_batch_size=variable_batch_size,
            group=self._pg,
            codecs=self._codecs,
        )
        return SequenceEmbeddingsAwaitable(tensor_awaitable, unbucketize_permute_tensor, local_embs.shape[1])


# ---- inference: all devices of one process -> one device --------------------------------------------
class EmbeddingsAllToOne(nn.Module):
    """Concatenate per-device pooled outputs ``[B, D_r]`` on ``device`` along ``cat_dim``."""

    def __init__(self, device: torch.device, world_size: int, cat_dim: int) -> None:
        super().__init__()
        self._device = device
        self._world_size = world_size
        self._cat_dim = cat_dim

    def forward(self, tensors: List[torch.Tensor]) -> torch.Tensor:
        assert len(tensors) <= self._world_size
        nonempty = [t for t in tensors if t.numel() > 0] or tensors
        return torch.cat([t.to(self._device, non_blocking=True) for t in nonempty], dim=self._cat_dim)

    def set_device(self, device_str: str) -> None:
        self._device = torch.device(device_str)


class MergePooledEmbeddingsModule(nn.Module):
    """Brings per-device tensors to one device and concatenates them along ``cat_dim``; a serving runtime can retarget it with
    ``set_device`` after the model was loaded (``torchrec/distributed/dist_data.py:185`` of the reference)."""

    def __init__(self, device: torch.device) -> None:
        super().__init__()
        self._device = device

    def set_device(self, device_str: str) -> None:
        self._device = torch.device(device_str)

    def forward(self, tensors: List[torch.Tensor], cat_dim: int) -> torch.Tensor:
        return torch.cat([t.to(self._device, non_blocking=True) for t in tensors], dim=cat_dim)


class EmbeddingsAllToOneReduce(nn.Module):
    """Sum per-device partial outputs on ``device`` (row-wise inference)."""

    def __init__(self, device: torch.device, world_size: int) -> None:
        super().__init__()
        self._device = device
        self._world_size = world_size

    def forward(self, tensors: List[torch.Tensor]) -> torch.Tensor:
        acc = tensors[0].to(self._device, non_blocking=True)
        for t in tensors[1:]:
            acc = acc + t.to(self._device, non_blocking=True)
        return acc

    def set_device(self, device_str: str) -> None:
        self._device = torch.device(device_str)


class SeqEmbeddingsAllToOne(nn.Module):
    """Move per-device sequence outputs to ``device`` keeping them as a list."""

    def __init__(self, device: torch.device, world_size: int) -> None:
        super().__init__()
        self._device = device
        self._world_size = world_size

    def forward(self, tensors: List[torch.Tensor]) -> List[torch.Tensor]:
        return [t.to(self._device, non_blocking=True) for t in tensors]

    def set_device(self, device_str: str) -> None:
        self._device = torch.device(device_str)


class TensorAllToAllValuesAwaitable(Awaitable[torch.Tensor]):
    """Rows (or elements) of a dense tensor on their way to the ranks named by the splits; the collective is started in the
    constructor and ``wait()`` returns the received tensor ``[sum(output_splits), ...]``.  No gradient flows through it (ids and
    pool rows travel this way; use ``comm_ops.tensor_alltoall`` for a differentiable exchange).
    Counterpart of ``torchrec/distributed/dist_data.py:1720-1763``."""

    def __init__(self, pg: dist.ProcessGroup, input: torch.Tensor, input_splits: torch.Tensor, output_splits: torch.Tensor, device: torch.device) -> None:
        super().__init__()
        self._workers = pg.size()
        self._work = None
        if self._workers == 1:
            self._dist_values = input
            return
        out_rows = int(output_splits.sum())
        self._dist_values = torch.empty((out_rows,) + tuple(input.shape[1:]), device=device, dtype=input.dtype)
        self._work = dist.all_to_all_single(self._dist_values, input.contiguous(), output_split_sizes=output_splits.tolist(),
                                            input_split_sizes=input_splits.tolist(), group=pg, async_op=True)

    def _wait_impl(self) -> torch.Tensor:
        if self._work is not None:
            self._work.wait()
        return self._dist_values


class TensorAllToAllSplitsAwaitable(Awaitable[TensorAllToAllValuesAwaitable]):
    """First stage of a dense-tensor all-to-all: every rank tells every other how many rows it will send; ``wait()`` starts the
    value exchange with the received counts and returns its awaitable (``torchrec/distributed/dist_data.py:1766-1810``)."""

    def __init__(self, pg: dist.ProcessGroup, input: torch.Tensor, splits: torch.Tensor, device: torch.device) -> None:
        super().__init__()
        self._workers = pg.size()
        self._pg, self._device, self._input, self._input_splits = pg, device, input, splits
        self._work = None
        if self._workers == 1:
            self._output_splits = splits
            return
        self._output_splits = torch.empty([self._workers], device=device, dtype=splits.dtype)
        self._work = dist.all_to_all_single(self._output_splits, splits.to(device), group=pg, async_op=True)

    def _wait_impl(self) -> TensorAllToAllValuesAwaitable:
        if self._work is not None:
            self._work.wait()
        return TensorAllToAllValuesAwaitable(self._pg, self._input, self._input_splits, self._output_splits, self._device)


class TensorAllToAll(nn.Module):
    """Redistribute a dense ``[n, ...]`` tensor whose rows are grouped by destination rank: ``forward(local_tensor, splits)`` with
    ``splits[r]`` rows for rank ``r`` returns the two-stage awaitable (counts, then values)."""

    def __init__(self, pg: dist.ProcessGroup) -> None:
        super().__init__()
        self._pg = pg

    def forward(self, local_tensor: torch.Tensor, splits: torch.Tensor) -> TensorAllToAllSplitsAwaitable:
        if not isinstance(splits, torch.Tensor):
            splits = torch.tensor(splits, dtype=torch.int64)
        return TensorAllToAllSplitsAwaitable(self._pg, local_tensor, splits, local_tensor.device)


class TensorValuesAllToAll(nn.Module):
    """The second stage on its own, for callers that already know both sides' counts."""

    def __init__(self, pg: dist.ProcessGroup) -> None:
        super().__init__()
        self._pg = pg

    def forward(self, input: torch.Tensor, input_splits: torch.Tensor, output_splits: torch.Tensor) -> TensorAllToAllValuesAwaitable:
        as_tensor = lambda x: x if isinstance(x, torch.Tensor) else torch.tensor(x, dtype=torch.int64)
        return TensorAllToAllValuesAwaitable(self._pg, input, as_tensor(input_splits), as_tensor(output_splits), input.device)


class JaggedTensorAllToAll(Awaitable):
    """Redistribute a ``JaggedTensor`` whose rows are grouped by destination rank."""

    def __init__(self, jt, num_items_to_send: torch.Tensor, num_items_to_receive: torch.Tensor, pg: dist.ProcessGroup) -> None:
        super().__init__()
        self._jt = jt
        self._pg = pg
        self._send = num_items_to_send.tolist()
        self._recv = num_items_to_receive.tolist()

    def _wait_impl(self):
        from torchrec_b200.sparse.jagged_tensor import JaggedTensor

        W = self._pg.size()
        lengths = self._jt.lengths()
        out_lengths = lengths.new_empty(sum(self._recv))
        dist.all_to_all_single(out_lengths, lengths.contiguous(), output_split_sizes=self._recv, input_split_sizes=self._send, group=self._pg)
        off = self._jt.offsets().tolist()
        send_vals, s = [], 0
        for n in self._send:
            send_vals.append(off[s + n] - off[s])
            s += n
        cs = [0] + list(itertools.accumulate(self._recv))
        ol = out_lengths.tolist()
        recv_vals = [sum(ol[cs[r]: cs[r + 1]]) for r in range(W)]
        values = self._jt.values()
        out_values = values.new_empty((sum(recv_vals),) + tuple(values.shape[1:]))
        dist.all_to_all_single(out_values, values.contiguous(), output_split_sizes=recv_vals, input_split_sizes=send_vals, group=self._pg)
        return JaggedTensor(values=out_values, lengths=out_lengths)
