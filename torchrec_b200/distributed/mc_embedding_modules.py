"""Sharded embedding collections behind managed collision (pooled and sequence form share this base).
Counterpart of ``torchrec/distributed/mc_embedding_modules.py:62``, ``mc_embeddingbag.py:52``, ``mc_embedding.py:67``."""
from __future__ import annotations

from typing import Any, Dict, Iterator, List, Optional, Tuple, Type

import torch
from torch import nn
from torch.nn.parallel import DistributedDataParallel

from torchrec_b200.distributed.embedding import EmbeddingCollectionContext, EmbeddingCollectionSharder, ShardedEmbeddingCollection
from torchrec_b200.distributed.embedding_types import BaseEmbeddingSharder, KJTList, ShardedEmbeddingModule
from torchrec_b200.distributed.embeddingbag import EmbeddingBagCollectionContext, EmbeddingBagCollectionSharder, ShardedEmbeddingBagCollection
from torchrec_b200.distributed.mc_modules import ShardedManagedCollisionCollection
from torchrec_b200.distributed.types import Awaitable, LazyAwaitable, NoWait, ParameterSharding, QuantizedCommCodecs, ShardingEnv, ShardingType
from torchrec_b200.modules.mc_embedding_modules import ManagedCollisionEmbeddingBagCollection, ManagedCollisionEmbeddingCollection
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class _ManagedCollisionFields:
    """What a managed-collision step adds to the context of the wrapped collection: the remapped ids per sharding (returned to the
    caller when asked for), the plan for sending them back to the requesting ranks, and the rows evicted in this step."""

    def _init_mc_fields(self, evictions_per_table: Optional[Dict[str, Optional[torch.Tensor]]] = None,
                        remapped_kjt: Optional[KJTList] = None) -> None:
        self.evictions_per_table = evictions_per_table
        self.remapped_kjt = remapped_kjt
        self.id_return_plan = None
        self.id_return_keys = None

    def _record_mc_stream(self, stream: torch.Stream) -> None:
        if self.evictions_per_table:
            for value in self.evictions_per_table.values():
                if value is not None and value.is_cuda:
                    value.record_stream(stream)
        if self.remapped_kjt is not None:
            for kjt in (self.remapped_kjt if isinstance(self.remapped_kjt, (list, KJTList)) else [self.remapped_kjt]):
                kjt.record_stream(stream)


class ManagedCollisionEmbeddingBagCollectionContext(EmbeddingBagCollectionContext, _ManagedCollisionFields):
    """Context of one step of a sharded ``ManagedCollisionEmbeddingBagCollection`` (``torchrec/distributed/mc_embeddingbag.py:36-49``)."""

    def __init__(self, sharding_contexts=None, inverse_indices=None, variable_batch_per_feature: bool = False, divisor=None,
                 evictions_per_table: Optional[Dict[str, Optional[torch.Tensor]]] = None, remapped_kjt: Optional[KJTList] = None) -> None:
        super().__init__(sharding_contexts, inverse_indices, variable_batch_per_feature, divisor)
        self._init_mc_fields(evictions_per_table, remapped_kjt)

    def record_stream(self, stream: torch.Stream) -> None:
        super().record_stream(stream)
        self._record_mc_stream(stream)


class ManagedCollisionEmbeddingCollectionContext(EmbeddingCollectionContext, _ManagedCollisionFields):
    """Context of one step of a sharded ``ManagedCollisionEmbeddingCollection`` (``torchrec/distributed/mc_embedding.py:41-64``)."""

    def __init__(self, sharding_contexts=None, input_features=None, reverse_indices=None,
                 evictions_per_table: Optional[Dict[str, Optional[torch.Tensor]]] = None, remapped_kjt: Optional[KJTList] = None) -> None:
        super().__init__(sharding_contexts, input_features, reverse_indices)
        self._init_mc_fields(evictions_per_table, remapped_kjt)

    def record_stream(self, stream: torch.Stream) -> None:
        super().record_stream(stream)
        self._record_mc_stream(stream)


class BaseShardedManagedCollisionEmbeddingCollection(ShardedEmbeddingModule):
    _context_type: Type[Any] = ManagedCollisionEmbeddingBagCollectionContext

    def __init__(self, module: nn.Module, table_name_to_parameter_sharding: Dict[str, ParameterSharding], e_sharder: BaseEmbeddingSharder, env: ShardingEnv,
                 device: torch.device, module_fqn: Optional[str] = None) -> None:
        super().__init__()
        self._device, self._env = device, env
        self._return_remapped_features = module._return_remapped_features
        self._embedding_module = e_sharder.shard(module._embedding_module, table_name_to_parameter_sharding, env=env, device=device,
                                                 module_fqn=(module_fqn + "._embedding_module") if module_fqn else None)
        if hasattr(self._embedding_module, "disable_fused_engine"):
            self._embedding_module.disable_fused_engine()  # ids are remapped on the owning rank between input dist and lookup
        self._managed_collision_collection = ShardedManagedCollisionCollection(module._managed_collision_collection, table_name_to_parameter_sharding, env, device)
        sizes = self._managed_collision_collection.table_input_sizes()
        buckets = self._managed_collision_collection.table_total_num_buckets()
        for sharding in self._embedding_module._embedding_shardings:
            sharding._table_hash_size_override = sizes      # row blocks follow the collision module's input id space
            sharding._keep_original_indices = True         # the owning rank remaps the raw id
            if buckets is not None:
                sharding._table_total_num_buckets_override = buckets
        self._lookups = self._embedding_module._lookups
        self._init_bounds = {c.name: (c.get_weight_init_min(), c.get_weight_init_max()) for c in self._managed_collision_collection._embedding_configs}

    def input_dist(self, ctx, features: KeyedJaggedTensor) -> Awaitable[Awaitable[KJTList]]:
        features = self._managed_collision_collection.preprocess(features)
        pending = self._embedding_module.input_dist(ctx, features)
        if self._return_remapped_features and self._env.world_size > 1:
            ctx.id_return_plan = self._plan_id_return(features)
            ctx.id_return_keys = list(features.keys())
        return pending

    # ---- remapped ids travel back to the rank that asked ------------------------------------------------------------------
    @torch.no_grad()
    def _plan_id_return(self, features: KeyedJaggedTensor) -> List[Tuple[KeyedJaggedTensor, torch.Tensor, torch.Tensor]]:
        """Per sharding group: (this rank's features in the group's order, the position of every id in the bucketized order, the
        number of ids routed to every owner).  The bucketization is the input distribution's own, run once more with the
        permutation output switched on (the pooled distribution does not keep one)."""
        from torchrec_b200.distributed.embedding_sharding import bucketize_kjt_before_all2all

        em = self._embedding_module
        ordered = features.permute(em._features_order, em._features_order_tensor) if em._has_features_permute else features
        plans = []
        for dist_module, part in zip(em._input_dists, ordered.split(em._feature_splits)):
            assert not part.variable_stride_per_key(), "remapped ids are returned for fixed-batch inputs only"
            world = dist_module._world_size
            bucketized, position = bucketize_kjt_before_all2all(
                part, num_buckets=world, block_sizes=dist_module._feature_block_sizes_tensor,
                total_num_blocks=dist_module._feature_total_num_blocks_tensor if dist_module._has_multiple_blocks_per_shard else None,
                output_permute=True, keep_original_indices=True)
            plans.append((part, position, bucketized.lengths().view(world, -1).sum(1)))
        return plans

    def _return_ids(self, ctx) -> KeyedJaggedTensor:
        """Send every remapped id (global row number) from the rank that owns its row back to the rank whose batch it came from,
        in the order of that rank's input (``torchrec/distributed/mc_modules.py:173-960`` of the reference returns them
        through a sequence output distribution of width one)."""
        import torch.distributed as dist

        from torchrec_b200.ops import sparse_ops as sops

        world, pg = self._env.world_size, self._env.process_group
        groups = []
        for (part, position, routed), owned in zip(ctx.id_return_plan, ctx.remapped_kjt):
            n_keys = len(owned.keys())
            lengths = owned.lengths().view(n_keys, -1)
            assert lengths.shape[1] % world == 0, "remapped ids are returned for equal batch sizes per rank only"
            per_key_rank = lengths.view(n_keys, world, -1).sum(2)  # ids of (feature, requesting rank)
            rank_major = torch.arange(n_keys * world, device=lengths.device).view(n_keys, world).t().reshape(-1)
            _, outgoing, _ = sops.permute_2D_sparse_data(rank_major, per_key_rank.reshape(-1, 1), owned.values())
            send_counts, recv_counts = per_key_rank.sum(0).tolist(), routed.tolist()
            incoming = outgoing.new_empty(sum(recv_counts))
            dist.all_to_all_single(incoming, outgoing.contiguous(), recv_counts, send_counts, group=pg)
            groups.append(KeyedJaggedTensor(keys=part.keys(), values=incoming.index_select(0, position.to(torch.int64)), weights=part.weights_or_none(),
                                            lengths=part.lengths(), offsets=part._offsets, stride=part._stride))
        merged = groups[0] if len(groups) == 1 else KeyedJaggedTensor.concat(groups)
        wanted = ctx.id_return_keys
        if merged.keys() != wanted and sorted(merged.keys()) == sorted(wanted):
            merged = merged.permute([merged.keys().index(k) for k in wanted])
        return merged

    @torch.no_grad()
    def _reset_rows(self, evictions: Dict[str, Optional[torch.Tensor]]) -> None:
        for table, rows in evictions.items():
            if rows is None or rows.numel() == 0:
                continue
            lo, hi = self._init_bounds[table]
            for _, w in self._embedding_module._model_parallel_name_to_local_shards.get(table, []):
                r = rows.to(w.device)
                w[r] = torch.empty(r.numel(), w.shape[1], device=w.device, dtype=torch.float32).uniform_(lo, hi).to(w.dtype)

    def _remap_list(self, ctx, dist_input: KJTList) -> KJTList:
        local, glob = [], []
        for features in dist_input:
            l, g = self._managed_collision_collection.remap(features)
            local.append(l)
            glob.append(g)
        ctx.evictions_per_table = self._managed_collision_collection.evict()
        self._reset_rows(ctx.evictions_per_table)
        ctx.remapped_kjt = glob
        return KJTList(local)

    def compute(self, ctx, dist_input: KJTList):
        return self._embedding_module.compute(ctx, self._remap_list(ctx, dist_input))

    def output_dist(self, ctx, output):
        return self._finish(ctx, self._embedding_module.output_dist(ctx, output))

    def compute_and_output_dist(self, ctx, input: KJTList):
        return self._finish(ctx, self._embedding_module.compute_and_output_dist(ctx, self._remap_list(ctx, input)))

    def _finish(self, ctx, lazy):
        if not self._return_remapped_features:
            return lazy, None
        if ctx.id_return_plan is not None:
            return lazy, NoWait(self._return_ids(ctx))
        # one rank: the remapped ids (global row numbers) are already where they were asked for
        return lazy, NoWait(ctx.remapped_kjt[0] if len(ctx.remapped_kjt) == 1 else ctx.remapped_kjt)

    def create_context(self):
        return self._context_type()

    def sharded_parameter_names(self, prefix: str = "") -> Iterator[str]:
        yield from self._embedding_module.sharded_parameter_names((prefix + "." if prefix else "") + "_embedding_module")

    def evict(self) -> Dict[str, Optional[torch.Tensor]]:
        return self._managed_collision_collection.evict()

    def open_slots(self) -> Dict[str, torch.Tensor]:
        return self._managed_collision_collection.open_slots()


class ShardedManagedCollisionEmbeddingBagCollection(BaseShardedManagedCollisionEmbeddingCollection):
    _context_type = ManagedCollisionEmbeddingBagCollectionContext

    @property
    def unsharded_module_type(self) -> Type[ManagedCollisionEmbeddingBagCollection]:
        return ManagedCollisionEmbeddingBagCollection


class ShardedManagedCollisionEmbeddingCollection(BaseShardedManagedCollisionEmbeddingCollection):
    _context_type = ManagedCollisionEmbeddingCollectionContext

    @property
    def unsharded_module_type(self) -> Type[ManagedCollisionEmbeddingCollection]:
        return ManagedCollisionEmbeddingCollection


class BaseManagedCollisionEmbeddingCollectionSharder(BaseEmbeddingSharder):
    """Sharder of a collection behind managed collision: wraps the sharder of the plain collection (row-wise only, since the owner
    of an id's row block is also the owner of its slot).  ``torchrec/distributed/mc_embedding_modules.py:336-390``."""

    _inner_sharder_type: Type[BaseEmbeddingSharder]
    _sharded_type: Type[BaseShardedManagedCollisionEmbeddingCollection]

    def __init__(self, e_sharder: Optional[BaseEmbeddingSharder] = None, qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None) -> None:
        super().__init__(qcomm_codecs_registry=qcomm_codecs_registry)
        self._e_sharder = e_sharder or self._inner_sharder_type(qcomm_codecs_registry=self.qcomm_codecs_registry)

    def shard(self, module, params: Dict[str, ParameterSharding], env: ShardingEnv, device: Optional[torch.device] = None, module_fqn: Optional[str] = None):
        device = device if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        return self._sharded_type(module, params, self._e_sharder, env, device, module_fqn)

    @property
    def fused_params(self) -> Optional[Dict[str, Any]]:
        return self._e_sharder.fused_params

    def shardable_parameters(self, module) -> Dict[str, nn.Parameter]:
        return self._e_sharder.shardable_parameters(module._embedding_module)

    def sharding_types(self, compute_device_type: str) -> List[str]:
        return [ShardingType.ROW_WISE.value]


class ManagedCollisionEmbeddingBagCollectionSharder(BaseManagedCollisionEmbeddingCollectionSharder):
    _inner_sharder_type = EmbeddingBagCollectionSharder
    _sharded_type = ShardedManagedCollisionEmbeddingBagCollection

    @property
    def module_type(self) -> Type[ManagedCollisionEmbeddingBagCollection]:
        return ManagedCollisionEmbeddingBagCollection


class ManagedCollisionEmbeddingCollectionSharder(BaseManagedCollisionEmbeddingCollectionSharder):
    _inner_sharder_type = EmbeddingCollectionSharder
    _sharded_type = ShardedManagedCollisionEmbeddingCollection

    @property
    def module_type(self) -> Type[ManagedCollisionEmbeddingCollection]:
        return ManagedCollisionEmbeddingCollection
