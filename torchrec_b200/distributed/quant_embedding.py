"""Sharded quantized ``EmbeddingCollection`` (sequence embeddings) for single-process multi-device inference; table-wise, row-wise
or column-wise placement, synchronous forward returning ``Dict[feature, JaggedTensor]`` (cf. ``torchrec/distributed/quant_embedding.py:549``)."""
from __future__ import annotations

import copy
from typing import Any, Dict, List, Optional, Type

import torch
from torch import nn

from torchrec_b200.distributed.embedding_types import BaseQuantEmbeddingSharder
from torchrec_b200.distributed.quant_embeddingbag import _device_for
from torchrec_b200.distributed.types import ParameterSharding, ShardingEnv, ShardingType
from torchrec_b200.distributed.quant_input_dist import (  # noqa: F401  (also the reference's import paths for these)
    ShardedQuantEcInputDist, create_infer_embedding_sharding, get_device_for_first_shard_from_sharding_infos, get_device_from_parameter_sharding, get_device_from_sharding_infos,
)
from torchrec_b200.distributed.quant_state import ShardedQuantEmbeddingModuleState
from torchrec_b200.quant.embedding_modules import EmbeddingCollection as QuantEmbeddingCollection
from torchrec_b200.quant.embedding_modules import QuantManagedCollisionEmbeddingCollection
from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor


class ShardedQuantEmbeddingCollection(ShardedQuantEmbeddingModuleState, nn.Module):
    """Sequence (unpooled) quantized lookups over the local devices.  ``table_wise``: whole table on ``ranks[0]``.  ``row_wise``: equal
    row blocks over all devices; ids are bucketized by block, every device returns the rows of its ids, and the rows are put back in
    request order.  ``column_wise``: one column range per entry of ``ranks`` (distinct devices); the ranges of every id are
    concatenated."""

    def __init__(self, module: QuantEmbeddingCollection, table_name_to_parameter_sharding: Dict[str, ParameterSharding], env: ShardingEnv,
                 fused_params: Optional[Dict[str, Any]] = None, device: Optional[torch.device] = None) -> None:
        super().__init__()
        from torchrec_b200.ops.quant_ops import BITS

        self._configs = module.embedding_configs()
        self._need_indices = module.need_indices()
        self._world_size = env.world_size
        self._device_type = (device.type if device is not None else ("cuda" if torch.cuda.is_available() else "cpu"))
        self._out_device = device if device is not None else _device_for(0, self._device_type)
        W = self._world_size
        by_rank: List[List[Any]] = [[] for _ in range(W)]
        rw: List[List[Any]] = [[] for _ in range(W)]
        cw: Dict[str, List[Any]] = {}  # "<rank>_<width>" -> local configs
        slices: Dict[Any, torch.Tensor] = {}
        self._rw_tables: List[Any] = []
        self._cw_tables: List[Any] = []  # (config, ranks, width)
        for cfg in self._configs:
            ps = table_name_to_parameter_sharding[cfg.name]
            packed = module.embeddings[cfg.name].weight
            bits = BITS[cfg.data_type]
            if ps.sharding_type == ShardingType.TABLE_WISE.value:
                by_rank[ps.ranks[0]].append(cfg)
            elif ps.sharding_type == ShardingType.ROW_WISE.value:
                block = (cfg.num_embeddings + W - 1) // W
                self._rw_tables.append((cfg, block))
                for r in range(W):
                    rows = max(0, min(block, cfg.num_embeddings - r * block))
                    local = copy.deepcopy(cfg)
                    local.num_embeddings = max(rows, 1)
                    rw[r].append(local)
                    slices[("rw", r, cfg.name)] = packed[r * block: r * block + rows] if rows > 0 else packed.new_zeros(1, packed.shape[1])
            elif ps.sharding_type == ShardingType.COLUMN_WISE.value:
                ranks = list(ps.ranks)
                if len(set(ranks)) != len(ranks) or cfg.embedding_dim % len(ranks):
                    raise ValueError(f"{cfg.name}: column-wise shards need distinct devices and a dim divisible by their count (ranks {ranks}, dim {cfg.embedding_dim})")
                width = cfg.embedding_dim // len(ranks)
                payload = cfg.embedding_dim * bits // 8
                self._cw_tables.append((cfg, ranks, width))
                for j, r in enumerate(ranks):
                    local = copy.deepcopy(cfg)
                    local.embedding_dim = width
                    cw.setdefault(f"{r}_{width}", []).append(local)
                    cols = packed[:, j * width * bits // 8: (j + 1) * width * bits // 8]
                    slices[("cw", r, cfg.name)] = torch.cat([cols, packed[:, payload:]], dim=1) if bits < 16 else cols
            else:
                raise ValueError(f"quantized inference sharding supports table_wise, row_wise and column_wise placement, got {ps.sharding_type} for {cfg.name}")

        def make(cfgs: List[Any], rank: int, kind: Optional[str]) -> nn.Module:
            dev = _device_for(rank, self._device_type)
            shard = QuantEmbeddingCollection(copy.deepcopy(cfgs), dev, need_indices=False if kind else module.need_indices(), output_dtype=module.output_dtype())
            for cfg in cfgs:
                src = slices[(kind, rank, cfg.name)] if kind else module.embeddings[cfg.name].weight
                shard.embeddings[cfg.name].weight.copy_(src.to(dev))
            # shared-feature names must match the unsharded module's (feature@table)
            shard._name_of = {k: v for k, v in module._name_of.items() if k.split(":")[0] in {c.name for c in cfgs}}
            return shard

        self._shards = nn.ModuleList([make(cfgs, r, None) if cfgs else nn.Identity() for r, cfgs in enumerate(by_rank)])
        self._feature_names_per_rank: List[List[str]] = [[f for c in cfgs for f in c.feature_names] for cfgs in by_rank]
        self._rw_shards = nn.ModuleList([make(cfgs, r, "rw") if cfgs else nn.Identity() for r, cfgs in enumerate(rw)])
        self._cw_shards = nn.ModuleDict({key: make(cfgs, int(key.split("_")[0]), "cw") for key, cfgs in cw.items()})
        self._cw_features: Dict[str, List[str]] = {key: [f for c in cfgs for f in c.feature_names] for key, cfgs in cw.items()}
        self._rw_feature_names: List[str] = [f for cfg, _ in self._rw_tables for f in cfg.feature_names]
        assert len(set(self._rw_feature_names)) == len(self._rw_feature_names), "a feature may feed only one row-wise sequence table"
        self._rw_out_names: List[str] = [module._name_of[f"{cfg.name}:{f}"] for cfg, _ in self._rw_tables for f in cfg.feature_names]
        self.register_buffer("_rw_block_sizes", torch.tensor([b for cfg, b in self._rw_tables for _ in cfg.feature_names], dtype=torch.int64), persistent=False)
        self._name_of = dict(module._name_of)
        self._input_dist = ShardedQuantEcInputDist(
            self._world_size, self._device_type, dict(enumerate(self._feature_names_per_rank)), dict(self._cw_features),
            {key: int(key.split("_")[0]) for key in self._cw_features}, self._rw_feature_names, self._rw_block_sizes)
        self._init_quant_state("embeddings", {c.name: table_name_to_parameter_sharding[c.name].sharding_type for c in self._configs})

    def forward(self, features: KeyedJaggedTensor) -> Dict[str, JaggedTensor]:
        dist = self._input_dist(features)
        out: Dict[str, JaggedTensor] = {}
        for rank, local in dist.table_wise.items():
            for k, jt in self._shards[rank](local).items():
                out[k] = jt.to(self._out_device)
        if dist.row_wise:
            F = len(self._rw_feature_names)
            rw_in = dist.row_wise_request
            rows = []
            for rank, local in enumerate(dist.row_wise):
                got = self._rw_shards[rank](local)
                rows.extend(got[n].values().to(self._out_device, non_blocking=True) for n in self._rw_out_names)
            # bucketized order is (device, feature, sample): undo it to the request's (feature, sample) order
            ordered = torch.cat(rows).index_select(0, dist.unbucketize_permute.to(self._out_device).long())
            lengths = rw_in.lengths().view(F, -1).to(self._out_device)
            ids = rw_in.values().to(self._out_device).split(rw_in.length_per_key()) if self._need_indices else None
            for i, (name, piece) in enumerate(zip(self._rw_out_names, ordered.split(rw_in.length_per_key()))):
                out[name] = JaggedTensor(values=piece, lengths=lengths[i], weights=ids[i] if ids is not None else None)
        cw_out: Dict[str, Dict[str, JaggedTensor]] = {key: self._cw_shards[key](local) for key, local in dist.column_wise.items()}
        for cfg, ranks, width in self._cw_tables:
            per_rank = [cw_out[f"{r}_{width}"] for r in ranks]
            for f in cfg.feature_names:
                name = self._name_of[f"{cfg.name}:{f}"]
                vals = torch.cat([p[name].values().to(self._out_device, non_blocking=True) for p in per_rank], dim=1)
                ids = features[f].values().to(self._out_device) if self._need_indices else None
                out[name] = JaggedTensor(values=vals, lengths=per_rank[0][name].lengths().to(self._out_device), weights=ids)
        return out


class QuantEmbeddingCollectionSharder(BaseQuantEmbeddingSharder[QuantEmbeddingCollection]):
    def shard(self, module: QuantEmbeddingCollection, params: Dict[str, ParameterSharding], env: ShardingEnv,
              device: Optional[torch.device] = None, module_fqn: Optional[str] = None) -> ShardedQuantEmbeddingCollection:
        return ShardedQuantEmbeddingCollection(module, params, env, getattr(self, "fused_params", None), device)

    def shardable_parameters(self, module: QuantEmbeddingCollection) -> Dict[str, torch.Tensor]:
        return {name: m.weight for name, m in module.embeddings.items()}

    def sharding_types(self, compute_device_type: str) -> List[str]:
        return [ShardingType.TABLE_WISE.value, ShardingType.ROW_WISE.value, ShardingType.COLUMN_WISE.value]

    @property
    def module_type(self) -> Type[QuantEmbeddingCollection]:
        return QuantEmbeddingCollection


class ShardedQuantManagedCollisionEmbeddingCollection(ShardedQuantEmbeddingCollection):
    """Sharded form of the quantized managed-collision collection.  The id maps stay whole on the device that receives the
    request (a sorted id array per table: megabytes against gigabytes of rows), ids are remapped there and the remapped ids are
    then distributed like any others.  ``forward`` returns ``(embeddings, remapped KJT)``
    (``torchrec/distributed/quant_embedding.py:1003-1260``)."""

    def __init__(self, module: QuantManagedCollisionEmbeddingCollection, table_name_to_parameter_sharding: Dict[str, ParameterSharding],
                 env: ShardingEnv, fused_params: Optional[Dict[str, Any]] = None, device: Optional[torch.device] = None) -> None:
        super().__init__(module, table_name_to_parameter_sharding, env, fused_params, device)
        self._managed_collision_collection = module._managed_collision_collection
        self._return_remapped_features = module._return_remapped_features

    def forward(self, features: KeyedJaggedTensor):  # type: ignore[override]
        remapped = self._managed_collision_collection(features)
        return super().forward(remapped), remapped


class QuantManagedCollisionEmbeddingCollectionSharder(BaseQuantEmbeddingSharder[QuantManagedCollisionEmbeddingCollection]):
    def shard(self, module: QuantManagedCollisionEmbeddingCollection, params: Dict[str, ParameterSharding], env: ShardingEnv,
              device: Optional[torch.device] = None, module_fqn: Optional[str] = None) -> ShardedQuantManagedCollisionEmbeddingCollection:
        return ShardedQuantManagedCollisionEmbeddingCollection(module, params, env, getattr(self, "fused_params", None), device)

    def shardable_parameters(self, module: QuantManagedCollisionEmbeddingCollection) -> Dict[str, torch.Tensor]:
        return {name: m.weight for name, m in module.embeddings.items()}

    def sharding_types(self, compute_device_type: str) -> List[str]:
        return [ShardingType.TABLE_WISE.value, ShardingType.ROW_WISE.value, ShardingType.COLUMN_WISE.value]

    @property
    def module_type(self) -> Type[QuantManagedCollisionEmbeddingCollection]:
        return QuantManagedCollisionEmbeddingCollection
