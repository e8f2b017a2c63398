"""Sharded in-training-pruning collections.  The tables are sharded like any embedding collection; after the input
distribution every rank remaps the ids it received onto the rows it holds (``GenericITEPModule`` for shards that hold whole
tables or column slices, ``RowwiseShardedITEPModule`` for row shards, whose input distribution is switched to cut the *unpruned*
id space into row blocks).  Counterpart of ``torchrec/distributed/itep_embeddingbag.py`` (``:70``, ``:349``)."""
from __future__ import annotations

from collections import defaultdict
from enum import Enum
from typing import Any, Dict, Iterator, List, Optional, Tuple, Type

import torch
from torch import nn
from torch.nn.parallel import DistributedDataParallel

from torchrec_b200.distributed.embedding import EmbeddingCollectionContext, EmbeddingCollectionSharder, ShardedEmbeddingCollection
from torchrec_b200.distributed.embedding_types import BaseEmbeddingSharder, KJTList, ShardedEmbeddingModule
from torchrec_b200.distributed.embeddingbag import EmbeddingBagCollectionContext, EmbeddingBagCollectionSharder, ShardedEmbeddingBagCollection
from torchrec_b200.distributed.types import Awaitable, LazyAwaitable, ParameterSharding, QuantizedCommCodecs, ShardingEnv, ShardingType
from torchrec_b200.modules.itep_embedding_modules import ITEPEmbeddingBagCollection, ITEPEmbeddingCollection
from torchrec_b200.modules.itep_modules import GenericITEPModule, RowwiseShardedITEPModule
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor, KeyedTensor


class ShardingTypeGroup(Enum):
    CW_GROUP = "column_wise_group"
    RW_GROUP = "row_wise_group"


SHARDING_TYPE_TO_GROUP: Dict[str, ShardingTypeGroup] = {
    ShardingType.ROW_WISE.value: ShardingTypeGroup.RW_GROUP,
    ShardingType.COLUMN_WISE.value: ShardingTypeGroup.CW_GROUP,
    ShardingType.TABLE_WISE.value: ShardingTypeGroup.CW_GROUP,
    ShardingType.TABLE_COLUMN_WISE.value: ShardingTypeGroup.CW_GROUP,
}


class ITEPEmbeddingBagCollectionContext(EmbeddingBagCollectionContext):
    is_reindexed: bool = False


class ITEPEmbeddingCollectionContext(EmbeddingCollectionContext):
    """Context of one step of a sharded ``ITEPEmbeddingCollection``: the sequence collection's context plus whether the ids were
    already moved to their pruned positions (``torchrec/distributed/itep_embeddingbag.py:311-314``)."""

    is_reindexed: bool = False


class _ShardedITEPBase(ShardedEmbeddingModule):
    """Shared by the pooled and the sequence form; ``self._inner`` is the sharded collection."""

    _INNER_ATTR = ""

    def _setup(self, inner: nn.Module, unsharded_itep: GenericITEPModule, params: Dict[str, ParameterSharding], env: ShardingEnv) -> None:
        self.register_buffer("_iter", torch.tensor(0, dtype=torch.int64, device=torch.device("cpu")))
        self.table_name_to_sharding_type = {t: ps.sharding_type for t, ps in params.items()}
        unpruned = unsharded_itep.table_name_to_unpruned_hash_sizes
        lookups: Dict[ShardingTypeGroup, List[nn.Module]] = defaultdict(list)
        sizes: Dict[ShardingTypeGroup, Dict[str, int]] = defaultdict(dict)
        for sharding_type, sharding, lookup in zip(inner._sharding_types, inner._embedding_shardings, inner._lookups):
            assert sharding_type in SHARDING_TYPE_TO_GROUP, f"in-training pruning does not support {sharding_type} tables"
            group = SHARDING_TYPE_TO_GROUP[sharding_type]
            lookups[group].append(lookup)
            lk = lookup.module if isinstance(lookup, DistributedDataParallel) else lookup
            for cfg in lk.grouped_configs:
                for t in cfg.embedding_tables:
                    if t.name in unpruned:
                        sizes[group][t.name] = unpruned[t.name]
            if group == ShardingTypeGroup.RW_GROUP:
                # the row blocks of the input distribution follow the unpruned id space
                sharding._table_hash_size_override = dict(unpruned)
        self._lookups = inner._lookups
        self._itep_module = GenericITEPModule(
            table_name_to_unpruned_hash_sizes=sizes[ShardingTypeGroup.CW_GROUP], lookups=lookups[ShardingTypeGroup.CW_GROUP],
            pruning_interval=unsharded_itep.pruning_interval, enable_pruning=unsharded_itep.enable_pruning, pg=env.process_group)
        self._rowwise_itep_module = RowwiseShardedITEPModule(
            table_name_to_sharding_type=self.table_name_to_sharding_type, table_name_to_unpruned_hash_sizes=sizes[ShardingTypeGroup.RW_GROUP],
            lookups=lookups[ShardingTypeGroup.RW_GROUP], pruning_interval=unsharded_itep.pruning_interval, enable_pruning=unsharded_itep.enable_pruning,
            pg=env.process_group)

    @property
    def _inner(self) -> nn.Module:
        return getattr(self, self._INNER_ATTR)

    def _reindex(self, dist_input: KJTList) -> KJTList:
        it = int(self._iter.item())
        out = []
        for sharding_type, features in zip(self._inner._sharding_types, dist_input):
            m = self._itep_module if SHARDING_TYPE_TO_GROUP[sharding_type] == ShardingTypeGroup.CW_GROUP else self._rowwise_itep_module
            out.append(m(features, it))
        return KJTList(out)

    def input_dist(self, ctx, features: KeyedJaggedTensor) -> Awaitable[Awaitable[KJTList]]:
        return self._inner.input_dist(ctx, features)

    def prefetch(self, dist_input: KJTList, forward_stream=None, ctx=None) -> None:
        assert ctx is not None
        reindexed = self._reindex(dist_input)
        for i, f in enumerate(reindexed):
            dist_input[i] = f
        ctx.is_reindexed = True
        self._inner.prefetch(dist_input, forward_stream, ctx)

    def compute(self, ctx, dist_input: KJTList):
        if not getattr(ctx, "is_reindexed", False):
            dist_input = self._reindex(dist_input)
            ctx.is_reindexed = True
        self._iter += 1
        return self._inner.compute(ctx, dist_input)

    def output_dist(self, ctx, output):
        return self._inner.output_dist(ctx, output)

    def compute_and_output_dist(self, ctx, input: KJTList):
        if not getattr(ctx, "is_reindexed", False):
            input = self._reindex(input)
            ctx.is_reindexed = True
        self._iter += 1
        return self._inner.compute_and_output_dist(ctx, input)

    _context_type: Type[Any] = ITEPEmbeddingBagCollectionContext

    def create_context(self):
        ctx = self._context_type()
        ctx.is_reindexed = False
        return ctx

    def sharded_parameter_names(self, prefix: str = "") -> Iterator[str]:
        yield from self._inner.sharded_parameter_names((prefix + "." if prefix else "") + self._INNER_ATTR)


class ShardedITEPEmbeddingBagCollection(_ShardedITEPBase):
    _INNER_ATTR = "_embedding_bag_collection"

    def __init__(self, module: ITEPEmbeddingBagCollection, table_name_to_parameter_sharding: Dict[str, ParameterSharding], ebc_sharder: EmbeddingBagCollectionSharder,
                 env: ShardingEnv, device: torch.device, module_fqn: Optional[str] = None) -> None:
        super().__init__()
        self._device, self._env = device, env
        self._embedding_bag_collection: ShardedEmbeddingBagCollection = ebc_sharder.shard(
            module._embedding_bag_collection, table_name_to_parameter_sharding, env=env, device=device,
            module_fqn=(module_fqn + "._embedding_bag_collection") if module_fqn else None)
        self._embedding_bag_collection.disable_fused_engine()  # ids are remapped between input dist and lookup
        self._setup(self._embedding_bag_collection, module._itep_module, table_name_to_parameter_sharding, env)

    @property
    def unsharded_module_type(self) -> Type[ITEPEmbeddingBagCollection]:
        return ITEPEmbeddingBagCollection


class ShardedITEPEmbeddingCollection(_ShardedITEPBase):
    _INNER_ATTR = "_embedding_collection"
    _context_type = ITEPEmbeddingCollectionContext

    def __init__(self, module: ITEPEmbeddingCollection, table_name_to_parameter_sharding: Dict[str, ParameterSharding], ec_sharder: EmbeddingCollectionSharder,
                 env: ShardingEnv, device: torch.device, module_fqn: Optional[str] = None) -> None:
        super().__init__()
        self._device, self._env = device, env
        self._embedding_collection: ShardedEmbeddingCollection = ec_sharder.shard(
            module._embedding_collection, table_name_to_parameter_sharding, env=env, device=device,
            module_fqn=(module_fqn + "._embedding_collection") if module_fqn else None)
        self._setup(self._embedding_collection, module._itep_module, table_name_to_parameter_sharding, env)

    @property
    def unsharded_module_type(self) -> Type[ITEPEmbeddingCollection]:
        return ITEPEmbeddingCollection


class ITEPEmbeddingBagCollectionSharder(BaseEmbeddingSharder[ITEPEmbeddingBagCollection]):
    def __init__(self, ebc_sharder: Optional[EmbeddingBagCollectionSharder] = None, qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None) -> None:
        super().__init__(qcomm_codecs_registry=qcomm_codecs_registry)
        self._ebc_sharder = ebc_sharder or EmbeddingBagCollectionSharder(qcomm_codecs_registry=self.qcomm_codecs_registry)

    def shard(self, module: ITEPEmbeddingBagCollection, params: Dict[str, ParameterSharding], env: ShardingEnv, device: Optional[torch.device] = None,
              module_fqn: Optional[str] = None) -> ShardedITEPEmbeddingBagCollection:
        device = device if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        return ShardedITEPEmbeddingBagCollection(module, params, ebc_sharder=self._ebc_sharder, env=env, device=device, module_fqn=module_fqn)

    @property
    def fused_params(self) -> Optional[Dict[str, Any]]:
        return self._ebc_sharder.fused_params

    def shardable_parameters(self, module: ITEPEmbeddingBagCollection) -> Dict[str, nn.Parameter]:
        return self._ebc_sharder.shardable_parameters(module._embedding_bag_collection)

    @property
    def module_type(self) -> Type[ITEPEmbeddingBagCollection]:
        return ITEPEmbeddingBagCollection

    def sharding_types(self, compute_device_type: str) -> List[str]:
        return list(SHARDING_TYPE_TO_GROUP.keys())


class ITEPEmbeddingCollectionSharder(BaseEmbeddingSharder[ITEPEmbeddingCollection]):
    def __init__(self, ec_sharder: Optional[EmbeddingCollectionSharder] = None, qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None) -> None:
        super().__init__(qcomm_codecs_registry=qcomm_codecs_registry)
        self._ec_sharder = ec_sharder or EmbeddingCollectionSharder(qcomm_codecs_registry=self.qcomm_codecs_registry)

    def shard(self, module: ITEPEmbeddingCollection, params: Dict[str, ParameterSharding], env: ShardingEnv, device: Optional[torch.device] = None,
              module_fqn: Optional[str] = None) -> ShardedITEPEmbeddingCollection:
        device = device if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        return ShardedITEPEmbeddingCollection(module, params, ec_sharder=self._ec_sharder, env=env, device=device, module_fqn=module_fqn)

    @property
    def fused_params(self) -> Optional[Dict[str, Any]]:
        return self._ec_sharder.fused_params

    def shardable_parameters(self, module: ITEPEmbeddingCollection) -> Dict[str, nn.Parameter]:
        return self._ec_sharder.shardable_parameters(module._embedding_collection)

    @property
    def module_type(self) -> Type[ITEPEmbeddingCollection]:
        return ITEPEmbeddingCollection

    def sharding_types(self, compute_device_type: str) -> List[str]:
        return [ShardingType.COLUMN_WISE.value, ShardingType.TABLE_WISE.value, ShardingType.ROW_WISE.value]
