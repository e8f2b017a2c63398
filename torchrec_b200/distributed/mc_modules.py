"""Sharded managed collision: every rank runs the collision modules of the table rows it holds.

Tables behind a managed-collision collection are row-wise sharded.  The input distribution of the embedding module is reused
with two changes: ids are cut into row blocks by the collision module's *input* id space (not by the table size) and travel
unchanged; the rank that receives them remaps them with its local collision module, whose output range is exactly the rank's
row shard, and looks the rows up locally.  Rows whose slot changed owner are re-initialised in the local shard.
Counterpart of ``torchrec/distributed/mc_modules.py`` (``ShardedManagedCollisionCollection`` ``:173``).
"""
from __future__ import annotations

import copy
from typing import Any, Dict, Iterator, List, Optional, Tuple, Type

import torch
import torch.distributed as dist
from torch import nn

from torchrec_b200.distributed.embedding_types import BaseEmbeddingSharder
from torchrec_b200.distributed.types import ParameterSharding, QuantizedCommCodecs, ShardedTensor, ShardingEnv, ShardingType
from torchrec_b200.modules.mc_modules import ManagedCollisionCollection, ManagedCollisionModule
from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor


class ShardedManagedCollisionCollection(nn.Module):
    """Local collision modules of this rank plus the routing facts the embedding module's input distribution needs."""

    def __init__(self, module: ManagedCollisionCollection, table_name_to_parameter_sharding: Dict[str, ParameterSharding], env: ShardingEnv, device: torch.device) -> None:
        super().__init__()
        self._env = env
        self._device = device
        self._rank = env.rank
        self._world_size = env.world_size
        self._embedding_configs = module.embedding_configs()
        self._table_to_features: Dict[str, List[str]] = {c.name: list(c.feature_names) for c in self._embedding_configs}
        self._feature_to_table: Dict[str, str] = {f: c.name for c in self._embedding_configs for f in c.feature_names}
        self.need_preprocess = module.need_preprocess
        self._unsharded: Dict[str, ManagedCollisionModule] = dict(module._managed_collision_modules.items())
        local: Dict[str, ManagedCollisionModule] = {}
        self._row_offset: Dict[str, int] = {}
        self._global_rows: Dict[str, int] = {}
        self._shard_bounds: Dict[str, List[int]] = {}
        for cfg in self._embedding_configs:
            ps = table_name_to_parameter_sharding[cfg.name]
            assert ps.sharding_type == ShardingType.ROW_WISE.value, f"managed collision needs row-wise tables, {cfg.name} is {ps.sharding_type}"
            shards = ps.sharding_spec.shards
            bounds = [s.shard_offsets[0] for s in shards] + [shards[-1].shard_offsets[0] + shards[-1].shard_sizes[0]]
            mine = shards[self._rank]
            off, rows = mine.shard_offsets[0], mine.shard_sizes[0]
            assert rows > 0, f"rank {self._rank} holds no row of {cfg.name}: managed collision needs a shard on every rank"
            mc = self._unsharded[cfg.name]
            local[cfg.name] = mc.rebuild_with_output_id_range((off, off + rows), output_segments=bounds, device=device)
            self._row_offset[cfg.name], self._global_rows[cfg.name], self._shard_bounds[cfg.name] = off, bounds[-1], bounds
        self._managed_collision_modules = nn.ModuleDict(local)
        self._register_state_dict_hook(self._post_state_dict_hook)
        self._register_load_state_dict_pre_hook(self._pre_load_state_dict_hook, with_module=True)

    # ---- routing ---------------------------------------------------------------------------------------------
    def table_input_sizes(self) -> Dict[str, int]:
        return {t: int(mc.input_size()) for t, mc in self._unsharded.items()}

    def table_total_num_buckets(self) -> Optional[Dict[str, int]]:
        out = {}
        for t, mc in self._unsharded.items():
            b = mc.buckets() if hasattr(mc, "buckets") and callable(getattr(mc, "buckets")) else None
            if b is not None and b != self._world_size and int(mc.input_size()) > 0:
                out[t] = int(b)
        return out if len(out) == len(self._unsharded) else None

    def preprocess(self, features: KeyedJaggedTensor) -> KeyedJaggedTensor:
        """Per-table id hashing into the collision module's input space, before the ids are routed."""
        if not self.need_preprocess or all(getattr(mc, "_input_hash_func", None) is None for mc in self._unsharded.values()):
            return features
        jt = features.to_dict()
        out: Dict[str, JaggedTensor] = {}
        for table, mc in self._unsharded.items():
            sub = {f: jt[f] for f in self._table_to_features[table] if f in jt}
            if sub:
                out.update(mc.preprocess(sub))
        values = torch.cat([out[k].values() if k in out else jt[k].values() for k in features.keys()])
        return KeyedJaggedTensor(keys=features.keys(), values=values, weights=features.weights_or_none(), lengths=features.lengths(), offsets=features._offsets,
                                 stride=features._stride)

    # ---- remap on the owning rank ------------------------------------------------------------------------------
    def remap(self, features: KeyedJaggedTensor) -> Tuple[KeyedJaggedTensor, KeyedJaggedTensor]:
        """``(ids as local rows of this rank's shards, ids as global rows)`` for a KJT that arrived through the input distribution."""
        jt = features.to_dict()
        remapped: Dict[str, JaggedTensor] = {}
        for table, mc in self._managed_collision_modules.items():
            sub = {f: jt[f] for f in self._table_to_features[table] if f in jt}
            if not sub:
                continue
            if self.training:
                sub = mc.profile(sub)
            remapped.update(mc.remap(sub))
        glob = torch.cat([remapped[k].values() for k in features.keys()]) if features.keys() else features.values()
        offs = torch.cat([torch.full_like(remapped[k].values(), self._row_offset[self._feature_to_table[k]]) for k in features.keys()]) if features.keys() else glob
        mk = lambda v: KeyedJaggedTensor(keys=features.keys(), values=v, weights=features.weights_or_none(), lengths=features.lengths(), offsets=features._offsets,
                                         stride=features._stride)
        return mk(glob - offs), mk(glob)

    def evict(self) -> Dict[str, Optional[torch.Tensor]]:
        """Rows to re-initialise, as local rows of this rank's shard."""
        out: Dict[str, Optional[torch.Tensor]] = {}
        for table, mc in self._managed_collision_modules.items():
            rows = mc.evict()
            out[table] = None if rows is None else rows - self._row_offset[table]
        return out

    def open_slots(self) -> Dict[str, torch.Tensor]:
        return {t: mc.open_slots() for t, mc in self._managed_collision_modules.items()}

    # ---- checkpoint: buffers with one entry per local slot become shards of a global tensor ----------------------
    def _slot_buffers(self, table: str) -> Iterator[Tuple[str, torch.Tensor]]:
        mc = self._managed_collision_modules[table]
        rows = mc.output_size()
        for name, buf in mc.named_buffers():
            if buf is not None and buf.dim() >= 1 and buf.shape[0] == rows:
                yield name, buf

    @staticmethod
    def _post_state_dict_hook(module: "ShardedManagedCollisionCollection", destination: Dict[str, Any], prefix: str, _local_metadata: Any) -> None:
        from torch.distributed._shard.sharded_tensor import Shard, ShardMetadata

        pg = module._env.process_group
        if pg is None or module._world_size == 1:
            return
        for table in module._managed_collision_modules.keys():
            bounds = module._shard_bounds[table]
            for name, buf in module._slot_buffers(table):
                key = f"{prefix}_managed_collision_modules.{table}.{name}"
                tail = list(buf.shape[1:])
                metas = [ShardMetadata(shard_offsets=[bounds[r]] + [0] * len(tail), shard_sizes=[bounds[r + 1] - bounds[r]] + tail,
                                       placement=f"rank:{r}/{module._device if module._device.type == 'cpu' else 'cuda:' + str(r)}") for r in range(module._world_size)]
                shard = Shard(tensor=buf.detach(), metadata=copy.deepcopy(metas[module._rank]))
                destination[key] = ShardedTensor._init_from_local_shards([shard], [module._global_rows[table]] + tail, process_group=pg)

    @staticmethod
    def _pre_load_state_dict_hook(module: "ShardedManagedCollisionCollection", state_dict: Dict[str, Any], prefix: str, *args: Any) -> None:
        for table in module._managed_collision_modules.keys():
            off = module._row_offset[table]
            for name, buf in module._slot_buffers(table):
                key = f"{prefix}_managed_collision_modules.{table}.{name}"
                src = state_dict.get(key)
                if src is None:
                    continue
                if isinstance(src, ShardedTensor):
                    state_dict[key] = src.local_shards()[0].tensor
                elif isinstance(src, torch.Tensor) and src.shape[0] == module._global_rows[table] and src.shape[0] != buf.shape[0]:
                    state_dict[key] = src[off: off + buf.shape[0]]


class ManagedCollisionCollectionSharder(BaseEmbeddingSharder[ManagedCollisionCollection]):
    """Builds the sharded collision collection that sits in front of a sharded embedding module.  It is used by the sharders of
    the managed-collision embedding collections; a collision collection is not sharded on its own (its slot tables follow the row
    blocks of the embedding tables they serve).  (``torchrec/distributed/mc_modules.py:843`` of the reference.)"""

    def __init__(self, qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None) -> None:
        super().__init__(qcomm_codecs_registry=qcomm_codecs_registry)

    def shard(self, module: ManagedCollisionCollection, params: Dict[str, ParameterSharding], env: ShardingEnv, embedding_shardings: Optional[List[Any]] = None,
              device: Optional[torch.device] = None, use_index_dedup: bool = False) -> ShardedManagedCollisionCollection:
        return ShardedManagedCollisionCollection(module, params, env, device if device is not None else torch.device("cpu"))

    def shardable_parameters(self, module: ManagedCollisionCollection) -> Dict[str, nn.Parameter]:
        raise NotImplementedError("a collision collection is sharded together with its embedding module")

    @property
    def module_type(self) -> Type[ManagedCollisionCollection]:
        return ManagedCollisionCollection

    def sharding_types(self, compute_device_type: str) -> List[str]:
        return [ShardingType.ROW_WISE.value]
