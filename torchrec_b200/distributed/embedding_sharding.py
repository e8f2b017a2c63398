"""Framework shared by all embedding shardings.

* ``bucketize_kjt_before_all2all``: row-wise bucketization of a KJT (ids -> owning row block).
* ``group_tables``: tables of a rank that can share one TBE (same dtype / pooling / weightedness /
  kernel / optimizer settings) are grouped.
* ``KJTListSplitsAwaitable`` / ``FusedKJTListSplitsAwaitable``: stage 1 of the input dist for a
  list of KJT all-to-alls; the fused variant exchanges the split sizes of every sharding type of
  every pipelined module in ONE collective.
* ABCs ``BaseSparseFeaturesDist`` / ``BaseEmbeddingDist`` / ``EmbeddingSharding``.

Counterpart of ``torchrec/distributed/embedding_sharding.py`` (``:219-287``, ``:503-623``,
``:630-926``, ``:988-1150``).
"""
from __future__ import annotations

import abc
import copy
from dataclasses import dataclass, field
from typing import Any, Dict, Generic, List, Optional, Tuple, TypeVar, Union

import torch
import torch.distributed as dist
from torch import nn

from torchrec_b200.distributed.dist_data import KJTAllToAllTensorsAwaitable, SplitsAllToAllAwaitable
from torchrec_b200.distributed.embedding_types import (
    BaseEmbeddingLookup,
    EmbeddingComputeKernel,
    FeatureShardingMixIn,
    GroupedEmbeddingConfig,
    KJTList,
    ListOfKJTList,
    ShardedEmbeddingTable,
)
from torchrec_b200.distributed.types import Awaitable, ParameterSharding, QuantizedCommCodecs, ShardMetadata
from torchrec_b200.modules.embedding_configs import DataType, EmbeddingTableConfig, PoolingType
from torchrec_b200.ops import sparse_ops as sops
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor
from torchrec_b200.streamable import Multistreamable

C = TypeVar("C", bound=Multistreamable)
F = TypeVar("F", bound=Multistreamable)
T = TypeVar("T")
W = TypeVar("W")


def _fx_wrap_tensor_to_device_dtype(t: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    return t.to(device=like.device, dtype=like.dtype)


def bucketize_kjt_before_all2all(
    kjt: KeyedJaggedTensor,
    num_buckets: int,
    block_sizes: torch.Tensor,
    total_num_blocks: Optional[torch.Tensor] = None,
    output_permute: bool = False,
    bucketize_pos: bool = False,
    block_bucketize_row_pos: Optional[List[torch.Tensor]] = None,
    keep_original_indices: bool = False,
) -> Tuple[KeyedJaggedTensor, Optional[torch.Tensor]]:
    """Split every bag by owning row block.

    The result has ``num_buckets * F`` keys (bucket-major: all features of bucket 0, then bucket
    1, ...), so a plain key-split all-to-all sends bucket ``r`` to rank ``r``; ids are made
    shard-local unless ``keep_original_indices``.  With ``output_permute`` the second result maps
    every input id to its slot in the bucketized order (needed to restore sequence order).
    """
    num_features = len(kjt.keys())
    assert block_sizes.numel() == num_features, f"Expecting block sizes for {num_features} features, but {block_sizes.numel()} received."
    block_sizes_new_type = _fx_wrap_tensor_to_device_dtype(block_sizes, kjt.values())
    bpf = None
    if kjt.variable_stride_per_key():
        bpf = torch.tensor(kjt.stride_per_key(), dtype=kjt.lengths().dtype, device=kjt.device())
    (bucketized_lengths, bucketized_indices, bucketized_weights, pos, unbucketize_permute) = sops.block_bucketize_sparse_features(
        kjt.lengths().view(-1),
        kjt.values(),
        bucketize_pos=bucketize_pos,
        sequence=output_permute,
        block_sizes=block_sizes_new_type,
        my_size=num_buckets,
        weights=kjt.weights_or_none(),
        batch_size_per_feature=bpf,
        max_B=-1,
        block_bucketize_pos=block_bucketize_row_pos,
        keep_orig_idx=keep_original_indices,
        total_num_blocks=None if total_num_blocks is None else _fx_wrap_tensor_to_device_dtype(total_num_blocks, kjt.values()),
    )
    spkpr = None
    stride = kjt.stride()
    if kjt.variable_stride_per_key():
        spkpr = kjt.stride_per_key_per_rank_tensor().repeat(num_buckets, 1)
        stride = None
    return (
        KeyedJaggedTensor(
            keys=_repeat_keys(kjt.keys(), num_buckets),
            values=bucketized_indices,
            weights=pos if bucketize_pos else bucketized_weights,
            lengths=bucketized_lengths.view(-1),
            offsets=None,
            stride=stride,
            stride_per_key_per_rank=spkpr,
            length_per_key=None,
            offset_per_key=None,
            index_per_key=None,
        ),
        unbucketize_permute,
    )


def bucketize_kjt_inference(
    kjt: KeyedJaggedTensor,
    num_buckets: int,
    block_sizes: torch.Tensor,
    total_num_buckets: Optional[torch.Tensor] = None,
    bucketize_pos: bool = False,
    block_bucketize_row_pos: Optional[List[torch.Tensor]] = None,
    is_sequence: bool = False,
    keep_original_indices: bool = False,
) -> Tuple[KeyedJaggedTensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
    """The row-wise split of a request at inference: like ``bucketize_kjt_before_all2all`` for a fixed batch, and for sequence
    features also ``bucket_mapping`` - the bucket every input id went to (what a caller needs to route per-id results back without
    the permutation).  Returns ``(bucketized KJT, unbucketize_permute or None, bucket_mapping or None)``.
    Counterpart of ``torchrec/distributed/embedding_sharding.py:307-389``."""
    out, unbucketize_permute = bucketize_kjt_before_all2all(
        kjt, num_buckets, block_sizes, total_num_blocks=total_num_buckets, output_permute=is_sequence, bucketize_pos=bucketize_pos,
        block_bucketize_row_pos=block_bucketize_row_pos, keep_original_indices=keep_original_indices)
    bucket_mapping = None
    if is_sequence and unbucketize_permute is not None:
        # position p of the bucketized order lies in bucket b when ends[b - 1] <= p < ends[b]
        ends = torch.cumsum(out.lengths().view(num_buckets, -1).sum(dim=1), 0)
        bucket_mapping = torch.searchsorted(ends, unbucketize_permute.to(ends.dtype), right=True).to(unbucketize_permute.dtype)
    return out, unbucketize_permute, bucket_mapping


def _repeat_keys(keys: List[str], n: int) -> List[str]:
    return list(keys) * n


def _get_weighted_avg_cache_load_factor(embedding_tables: List[ShardedEmbeddingTable]) -> Optional[float]:
    num, den = 0.0, 0.0
    for t in embedding_tables:
        clf = None if t.fused_params is None else t.fused_params.get("cache_load_factor")
        if clf is not None:
            sz = t.local_rows * t.local_cols
            num += clf * sz
            den += sz
    return None if den == 0 else num / den


def _get_grouping_fused_params(fused_params: Optional[Dict[str, Any]], name: str) -> Optional[Dict[str, Any]]:
    """Parameters that do not force separate TBEs are removed before tables are compared."""
    if fused_params is None:
        return None
    fp = copy.copy(fused_params)
    for k in ("cache_load_factor", "prefetch_pipeline", "enforce_hbm"):
        fp.pop(k, None)
    return fp


def _to_hashable(x: Any) -> Any:
    if isinstance(x, dict):
        return tuple(sorted((k, _to_hashable(v)) for k, v in x.items()))
    if isinstance(x, (list, tuple)):
        return tuple(_to_hashable(v) for v in x)
    try:
        hash(x)
        return x
    except TypeError:
        return repr(x)


def group_tables(tables_per_rank: List[List[ShardedEmbeddingTable]]) -> List[List[GroupedEmbeddingConfig]]:
    """Group the tables of every rank into TBEs; each group becomes one flat buffer and one kernel launch."""

    def _group_one(embedding_tables: List[ShardedEmbeddingTable]) -> List[GroupedEmbeddingConfig]:
        groups: Dict[Any, List[ShardedEmbeddingTable]] = {}
        order: List[Any] = []
        for table in embedding_tables:
            key = (
                table.data_type,
                table.pooling,
                table.is_weighted,
                table.has_feature_processor,
                table.compute_kernel,
                _to_hashable(_get_grouping_fused_params(table.fused_params, table.name)),
                # unpooled TBEs need one dim; pooled ones may mix dims
                table.local_cols if table.pooling == PoolingType.NONE else 0,
                table.use_virtual_table,
            )
            if key not in groups:
                groups[key] = []
                order.append(key)
            groups[key].append(table)
        out: List[GroupedEmbeddingConfig] = []
        for key in order:
            tables = groups[key]
            fused_params = copy.copy(tables[0].fused_params) if tables[0].fused_params is not None else {}
            clf = _get_weighted_avg_cache_load_factor(tables)
            if clf is not None:
                fused_params["cache_load_factor"] = clf
            out.append(
                GroupedEmbeddingConfig(
                    data_type=key[0], pooling=key[1], is_weighted=key[2], has_feature_processor=key[3],
                    compute_kernel=key[4], embedding_tables=tables, fused_params=fused_params,
                )
            )
        return out

    return [_group_one(t) for t in tables_per_rank]


# ---- input-dist awaitables --------------------------------------------------------------------------
class KJTListAwaitable(Awaitable[KJTList]):
    """Waits on the payload all-to-alls of several KJTs and returns them as a ``KJTList``."""

    def __init__(self, awaitables: List[Awaitable[KeyedJaggedTensor]], ctx: C, module_fqn: Optional[str] = None, sharding_types: Optional[List[str]] = None) -> None:
        super().__init__()
        self.awaitables = awaitables
        self.ctx = ctx
        self._module_fqn = module_fqn
        self._sharding_types = sharding_types

    def _wait_impl(self) -> KJTList:
        kjts = [w.wait() for w in self.awaitables]
        _set_sharding_context_post_a2a(kjts, self.ctx)
        return KJTList(kjts)


def _set_sharding_context_post_a2a(kjts: List[KeyedJaggedTensor], ctx: C) -> None:
    for kjt, sharding_context in zip(kjts, getattr(ctx, "sharding_contexts", [])):
        if hasattr(sharding_context, "batch_size_per_rank_per_feature") and kjt.variable_stride_per_key() and kjt.stride_per_key_per_rank():
            strides = kjt.stride_per_key_per_rank()
            sharding_context.batch_size_per_rank_per_feature = [
                [strides[i][j] for i in range(len(strides))] for j in range(len(strides[0]))
            ]


def _set_sharding_context_intra_a2a(tensors_awaitables: List[Awaitable[KeyedJaggedTensor]], ctx: C) -> None:
    for awaitable, sharding_context in zip(tensors_awaitables, getattr(ctx, "sharding_contexts", [])):
        if isinstance(awaitable, KJTAllToAllTensorsAwaitable):
            if hasattr(sharding_context, "sparse_features_recat"):
                sharding_context.sparse_features_recat = awaitable._recat
            if hasattr(sharding_context, "input_splits") and "values" in awaitable._input_splits:
                sharding_context.input_splits = awaitable._input_splits["values"]
            if hasattr(sharding_context, "output_splits") and "values" in awaitable._output_splits:
                sharding_context.output_splits = awaitable._output_splits["values"]
            if hasattr(sharding_context, "batch_size_per_rank") and awaitable._stride_per_rank is not None:
                sharding_context.batch_size_per_rank = awaitable._stride_per_rank
                sharding_context.variable_batch_per_rank = len(set(awaitable._stride_per_rank)) > 1


def _split(flat_list: List[T], splits: List[int]) -> List[List[T]]:
    out, i = [], 0
    for s in splits:
        out.append(flat_list[i: i + s])
        i += s
    return out


class KJTListSplitsAwaitable(Awaitable[Awaitable[KJTList]], Generic[C]):
    """Stage 1 for the KJT all-to-alls of one module: waits on each splits exchange."""

    def __init__(self, awaitables: List[Awaitable[Awaitable[KeyedJaggedTensor]]], ctx: C, module_fqn: Optional[str] = None, sharding_types: Optional[List[str]] = None) -> None:
        super().__init__()
        self.awaitables = awaitables
        self.ctx = ctx
        self._module_fqn = module_fqn
        self._sharding_types = sharding_types

    def _wait_impl(self) -> KJTListAwaitable:
        tensors_awaitables = [w.wait() for w in self.awaitables]
        _set_sharding_context_intra_a2a(tensors_awaitables, self.ctx)
        return KJTListAwaitable(tensors_awaitables, self.ctx, self._module_fqn, self._sharding_types)


class FusedKJTListSplitsAwaitable(Awaitable[List[KJTListAwaitable]]):
    """ONE splits all-to-all for the input dists of several modules / sharding types on one process group."""

    def __init__(self, requests: List[KJTListSplitsAwaitable[C]], contexts: List[C], pg: Optional[dist.ProcessGroup]) -> None:
        super().__init__()
        self._contexts = contexts
        self._awaitables = [w for r in requests for w in r.awaitables]
        self._output_lengths = [len(r.awaitables) for r in requests]
        self._lengths = [
            (len(w._input_tensors) if w._input.variable_stride_per_key() else len(w._input_tensors) + 1)
            if hasattr(w, "_input_tensors") else 0
            for w in self._awaitables
        ]
        splits: List[List[int]] = []
        device = None
        for w in self._awaitables:
            if not hasattr(w, "_input_tensors"):
                continue
            splits.extend(w._input_splits)
            if not w._input.variable_stride_per_key():
                splits.append([w._input.stride()] * w._workers)
            device = w._device
        self._splits_awaitable = None
        if splits and pg is not None and pg.size() > 1:
            self._splits_awaitable = SplitsAllToAllAwaitable([list(s) for s in splits], pg, device=device)
        self._flat_splits = splits

    def _wait_impl(self) -> List[KJTListAwaitable]:
        if self._splits_awaitable is not None:
            output_splits = self._splits_awaitable.wait()
        else:
            output_splits = self._flat_splits
        splits_per_awaitable = _split(output_splits, self._lengths)
        tensors_awaitables = []
        for splits, w in zip(splits_per_awaitable, self._awaitables):
            if not splits:
                tensors_awaitables.append(w.wait())
                continue
            if w._input.variable_stride_per_key():
                out_splits, stride_per_rank = splits, None
            else:
                out_splits, stride_per_rank = splits[:-1], splits[-1]
            tensors_awaitables.append(
                KJTAllToAllTensorsAwaitable(
                    pg=w._pg, input=w._input, splits=w._splits, input_splits=w._input_splits, output_splits=out_splits,
                    input_tensors=w._input_tensors, labels=w._labels, keys=w._keys, device=w._device, stagger=w._stagger,
                    stride_per_rank=stride_per_rank,
                )
            )
        output = []
        for ta, ctx in zip(_split(tensors_awaitables, self._output_lengths), self._contexts):
            _set_sharding_context_intra_a2a(ta, ctx)
            output.append(KJTListAwaitable(ta, ctx))
        return output


class ListOfKJTListAwaitable(Awaitable[ListOfKJTList]):
    def __init__(self, awaitables: List[Awaitable[KJTList]]) -> None:
        super().__init__()
        self.awaitables = awaitables

    def _wait_impl(self) -> ListOfKJTList:
        return ListOfKJTList([w.wait() for w in self.awaitables])


class ListOfKJTListSplitsAwaitable(Awaitable[Awaitable[ListOfKJTList]]):
    def __init__(self, awaitables: List[Awaitable[Awaitable[KJTList]]]) -> None:
        super().__init__()
        self.awaitables = awaitables

    def _wait_impl(self) -> Awaitable[ListOfKJTList]:
        return ListOfKJTListAwaitable([w.wait() for w in self.awaitables])


# ---- contexts and ABCs --------------------------------------------------------------------------------
class EmbeddingShardingContext(Multistreamable):
    """Per-batch facts a sharding records during input dist for its output dist."""

    def __init__(self, batch_size_per_rank: Optional[List[int]] = None, batch_size_per_rank_per_feature: Optional[List[List[int]]] = None,
                 batch_size_per_feature_pre_a2a: Optional[List[int]] = None, variable_batch_per_feature: bool = False) -> None:
        super().__init__()
        self.batch_size_per_rank: List[int] = batch_size_per_rank if batch_size_per_rank is not None else []
        self.batch_size_per_rank_per_feature: List[List[int]] = batch_size_per_rank_per_feature if batch_size_per_rank_per_feature is not None else []
        self.batch_size_per_feature_pre_a2a: List[int] = batch_size_per_feature_pre_a2a if batch_size_per_feature_pre_a2a is not None else []
        self.variable_batch_per_feature: bool = variable_batch_per_feature
        self.variable_batch_per_rank: bool = False

    def record_stream(self, stream: torch.Stream) -> None:
        pass


class BaseSparseFeaturesDist(abc.ABC, nn.Module, Generic[F]):
    """Redistributes sparse inputs to the ranks that own the tables."""

    @abc.abstractmethod
    def forward(self, sparse_features: KeyedJaggedTensor) -> Union[Awaitable[Awaitable[F]], F]:
        ...


class BaseEmbeddingDist(abc.ABC, nn.Module, Generic[C, T, W]):
    """Redistributes lookup results to the ranks that own the samples."""

    @abc.abstractmethod
    def forward(self, local_embs: T, sharding_ctx: Optional[C] = None) -> Union[Awaitable[W], W]:
        ...


class EmbeddingSharding(abc.ABC, Generic[C, F, T, W], FeatureShardingMixIn):
    """One sharding strategy: knows how to build its input dist, lookup and output dist."""

    def __init__(self, qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None) -> None:
        self._qcomm_codecs_registry = qcomm_codecs_registry

    @property
    def qcomm_codecs_registry(self) -> Optional[Dict[str, QuantizedCommCodecs]]:
        return self._qcomm_codecs_registry

    @abc.abstractmethod
    def create_input_dist(self, device: Optional[torch.device] = None) -> BaseSparseFeaturesDist[F]:
        ...

    @abc.abstractmethod
    def create_output_dist(self, device: Optional[torch.device] = None) -> BaseEmbeddingDist[C, T, W]:
        ...

    @abc.abstractmethod
    def create_lookup(self, device: Optional[torch.device] = None, fused_params: Optional[Dict[str, Any]] = None, feature_processor=None) -> BaseEmbeddingLookup[F, T]:
        ...

    @abc.abstractmethod
    def embedding_dims(self) -> List[int]:
        ...

    @abc.abstractmethod
    def embedding_shard_metadata(self) -> List[Optional[ShardMetadata]]:
        ...

    @abc.abstractmethod
    def embedding_names(self) -> List[str]:
        ...

    @abc.abstractmethod
    def embedding_names_per_rank(self) -> List[List[str]]:
        ...

    def embedding_tables(self) -> List[ShardedEmbeddingTable]:
        raise NotImplementedError

    def uncombined_embedding_dims(self) -> List[int]:
        return self.embedding_dims()

    def uncombined_embedding_names(self) -> List[str]:
        return self.embedding_names()


@dataclass
class EmbeddingShardingInfo:
    embedding_config: EmbeddingTableConfig
    param_sharding: ParameterSharding
    param: torch.Tensor
    fused_params: Optional[Dict[str, Any]] = None
