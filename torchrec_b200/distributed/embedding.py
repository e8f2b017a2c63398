"""Sharded ``EmbeddingCollection`` (unpooled / sequence embeddings).

Input dist as for pooled tables (plus optional per-feature id de-duplication), lookup returns one row
per id, and the sequence all-to-all sends every row back to the rank and position that asked for it.
The result is ``Dict[feature, JaggedTensor]`` exactly like the unsharded module; column-wise shards of
a table are concatenated along the embedding dim.

Counterpart of ``torchrec/distributed/embedding.py`` (``ShardedEmbeddingCollection`` ``:397``, index
dedup ``:1329``, sharder ``:1675``).
"""
from __future__ import annotations

import copy
from collections import OrderedDict, defaultdict
from typing import Any, Dict, Iterator, List, Optional, Tuple, Type, Union

import torch
import torch.distributed as dist
from torch import nn
from torch.autograd.profiler import record_function
from torch.nn.parallel import DistributedDataParallel

from torchrec_b200.distributed.batched_embedding_kernel import TableBatchedEmbeddingSlice, get_state_dict
from torchrec_b200.distributed.embedding_sharding import EmbeddingSharding, EmbeddingShardingInfo, KJTListSplitsAwaitable
from torchrec_b200.distributed.embedding_types import BaseEmbeddingSharder, EmbeddingComputeKernel, KJTList, ShardedEmbeddingModule
from torchrec_b200.distributed.sharding.cw_sequence_sharding import CwSequenceEmbeddingSharding
from torchrec_b200.distributed.sharding.dp_sequence_sharding import DpSequenceEmbeddingSharding
from torchrec_b200.distributed.sharding.rw_sequence_sharding import RwSequenceEmbeddingSharding
from torchrec_b200.distributed.sharding.rw_sharding import RwSparseFeaturesDist
from torchrec_b200.distributed.sharding.sequence_sharding import SequenceShardingContext
from torchrec_b200.distributed.sharding.tw_sequence_sharding import TwSequenceEmbeddingSharding
from torchrec_b200.distributed.types import (
    Awaitable,
    EmbeddingModuleShardingPlan,
    LazyAwaitable,
    ParameterSharding,
    QuantizedCommCodecs,
    ShardedTensor,
    ShardingEnv,
    ShardingEnv2D,
    ShardingType,
)
from torchrec_b200.distributed.utils import (
    add_params_from_parameter_sharding,
    append_prefix,
    convert_to_fbgemm_types,
    merge_fused_params,
    optimizer_type_to_emb_opt_type,
)
from torchrec_b200.modules.embedding_configs import EmbeddingConfig, EmbeddingTableConfig, PoolingType
from torchrec_b200.modules.embedding_modules import EmbeddingCollection, EmbeddingCollectionInterface
from torchrec_b200.ops import sparse_ops as sops
from torchrec_b200.optim.fused import EmptyFusedOptimizer, FusedOptimizerModule
from torchrec_b200.optim.keyed import CombinedOptimizer, KeyedOptimizer
from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor
from torchrec_b200.streamable import Multistreamable

EC_INDEX_DEDUP: bool = False


def get_ec_index_dedup() -> bool:
    return EC_INDEX_DEDUP


def set_ec_index_dedup(val: bool) -> None:
    """De-duplicate ids per feature before the input dist (smaller all-to-alls for repeated ids)."""
    global EC_INDEX_DEDUP
    EC_INDEX_DEDUP = val


def create_embedding_sharding(sharding_type: str, sharding_infos: List[EmbeddingShardingInfo], env: ShardingEnv,
                              device: Optional[torch.device] = None, qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None):
    if sharding_type == ShardingType.TABLE_WISE.value:
        return TwSequenceEmbeddingSharding(sharding_infos, env, device, qcomm_codecs_registry=qcomm_codecs_registry)
    if sharding_type == ShardingType.ROW_WISE.value:
        return RwSequenceEmbeddingSharding(sharding_infos, env, device, qcomm_codecs_registry=qcomm_codecs_registry)
    if sharding_type == ShardingType.DATA_PARALLEL.value:
        return DpSequenceEmbeddingSharding(sharding_infos, env, device)
    if sharding_type == ShardingType.COLUMN_WISE.value:
        return CwSequenceEmbeddingSharding(sharding_infos, env, device, qcomm_codecs_registry=qcomm_codecs_registry)
    raise ValueError(f"Sharding not supported {sharding_type}")


def construct_jagged_tensors(embeddings: torch.Tensor, features: KeyedJaggedTensor, embedding_names: List[str], need_indices: bool = False,
                             features_to_permute_indices: Optional[Dict[str, List[int]]] = None,
                             original_features: Optional[KeyedJaggedTensor] = None, reverse_indices: Optional[torch.Tensor] = None) -> Dict[str, JaggedTensor]:
    """Cut ``embeddings [sum L, D]`` (key-major like ``features``) into one ``JaggedTensor`` per embedding name;
    several entries with the same name are column shards and are concatenated along dim 1."""
    with record_function("## construct_jagged_tensors ##"):
        if original_features is not None:
            features = original_features
        if reverse_indices is not None:
            embeddings = torch.index_select(embeddings, 0, reverse_indices.to(torch.int64))
        ret: Dict[str, JaggedTensor] = {}
        lengths = features.lengths().view(-1, features.stride())
        length_per_key = features.length_per_key()
        values = features.values()
        lengths_tuple = torch.unbind(lengths, dim=0)
        embeddings_list = torch.split(embeddings, length_per_key, dim=0)
        values_list = torch.split(values, length_per_key) if need_indices else None
        key_indices: Dict[str, List[int]] = defaultdict(list)
        for i, key in enumerate(embedding_names):
            key_indices[key].append(i)
        for key, indices in key_indices.items():
            if features_to_permute_indices and key in features_to_permute_indices:
                perm = features_to_permute_indices[key]
                indices = [indices[p] for p in perm] if len(perm) == len(indices) else indices
            ret[key] = JaggedTensor(
                lengths=lengths_tuple[indices[0]],
                values=embeddings_list[indices[0]] if len(indices) == 1 else torch.cat([embeddings_list[i] for i in indices], dim=1),
                weights=values_list[indices[0]] if values_list is not None else None,
            )
        return ret


class EmbeddingCollectionContext(Multistreamable):
    def __init__(self, sharding_contexts: Optional[List[SequenceShardingContext]] = None, input_features: Optional[List[KeyedJaggedTensor]] = None,
                 reverse_indices: Optional[List[torch.Tensor]] = None) -> None:
        super().__init__()
        self.sharding_contexts: List[SequenceShardingContext] = sharding_contexts or []
        self.input_features: List[KeyedJaggedTensor] = input_features or []
        self.reverse_indices: List[torch.Tensor] = reverse_indices or []

    def record_stream(self, stream: torch.Stream) -> None:
        for ctx in self.sharding_contexts:
            ctx.record_stream(stream)
        for f in self.input_features:
            f.record_stream(stream)
        for r in self.reverse_indices:
            if r.is_cuda:
                r.record_stream(stream)


class EmbeddingCollectionAwaitable(LazyAwaitable[Dict[str, JaggedTensor]]):
    def __init__(self, awaitables_per_sharding: List[Awaitable[torch.Tensor]], features_per_sharding: List[KeyedJaggedTensor],
                 embedding_names_per_sharding: List[List[str]], ctx: EmbeddingCollectionContext, need_indices: bool = False,
                 features_to_permute_indices: Optional[Dict[str, List[int]]] = None) -> None:
        super().__init__()
        self._awaitables_per_sharding = awaitables_per_sharding
        self._features_per_sharding = features_per_sharding
        self._need_indices = need_indices
        self._features_to_permute_indices = features_to_permute_indices
        self._embedding_names_per_sharding = embedding_names_per_sharding
        self._ctx = ctx

    def _wait_impl(self) -> Dict[str, JaggedTensor]:
        jt_dict: Dict[str, JaggedTensor] = {}
        for i, (w, features, embedding_names) in enumerate(zip(self._awaitables_per_sharding, self._features_per_sharding, self._embedding_names_per_sharding)):
            original_features = self._ctx.input_features[i] if i < len(self._ctx.input_features) else None
            reverse_indices = self._ctx.reverse_indices[i] if i < len(self._ctx.reverse_indices) else None
            jt_dict.update(
                construct_jagged_tensors(
                    embeddings=w.wait(), features=features, embedding_names=embedding_names, need_indices=self._need_indices,
                    features_to_permute_indices=self._features_to_permute_indices, original_features=original_features,
                    reverse_indices=reverse_indices,
                )
            )
        return jt_dict
