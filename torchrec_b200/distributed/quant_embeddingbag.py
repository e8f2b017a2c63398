"""Sharded quantized ``EmbeddingBagCollection`` for inference: ONE process drives all devices.

Tables are placed table-wise, row-wise or column-wise following the module sharding plan; the request KJT is split by feature
(row-wise tables: also by row block) and copied to the owning devices, each device runs its quantized lookups, and the pooled
outputs are assembled on the output device in the key order of the unsharded module.  Synchronous ``forward`` (no awaitables),
as serving code expects.  Counterpart of ``torchrec/distributed/quant_embeddingbag.py:165-470`` and the inference dists of
``sharding/{tw,rw,cw}_sharding.py``.
"""
from __future__ import annotations

import copy
from typing import Any, Dict, List, Optional, Type

import torch
from torch import nn

from torchrec_b200.distributed.embedding_types import BaseQuantEmbeddingSharder
from torchrec_b200.distributed.types import ParameterSharding, ShardingEnv, ShardingType
from torchrec_b200.modules.embedding_configs import PoolingType
from torchrec_b200.distributed.quant_input_dist import (  # noqa: F401  (also the reference's import paths for these)
    ShardedQuantEbcInputDist, create_infer_embedding_bag_sharding, flatten_feature_lengths, get_device_for_first_shard_from_sharding_infos, get_device_from_parameter_sharding, get_device_from_sharding_infos,
)
from torchrec_b200.distributed.quant_state import ShardedQuantEmbeddingModuleState
from torchrec_b200.quant.embedding_modules import EmbeddingBagCollection as QuantEmbeddingBagCollection
from torchrec_b200.quant.embedding_modules import FeatureProcessedEmbeddingBagCollection as QuantFeatureProcessedEmbeddingBagCollection
from torchrec_b200.quant.embedding_modules import EmbeddingCollection as QuantEmbeddingCollection
from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor, KeyedTensor


def _device_for(rank: int, device_type: str) -> torch.device:
    return torch.device("cuda", rank) if device_type == "cuda" else torch.device(device_type)


class ShardedQuantEmbeddingBagCollection(ShardedQuantEmbeddingModuleState, nn.Module):
    """Placement per table: ``table_wise`` (whole table on ``ranks[0]``), ``row_wise`` (equal row blocks over all devices; ids are
    bucketized by block, every device pools its part, the parts are summed) or ``column_wise`` (one column range per entry of
    ``ranks``, all on distinct devices; every device pools its columns, the ranges are concatenated).  Quantized rows are cut
    without requantizing: a row block keeps whole rows, a column range keeps its payload bytes and a copy of the row's scale and
    bias."""

    def __init__(self, module: QuantEmbeddingBagCollection, table_name_to_parameter_sharding: Dict[str, ParameterSharding], env: ShardingEnv,
                 fused_params: Optional[Dict[str, Any]] = None, device: Optional[torch.device] = None) -> None:
        super().__init__()
        from torchrec_b200.ops.quant_ops import BITS

        self._configs = module.embedding_bag_configs()
        self._is_weighted = module.is_weighted()
        self._out_dtype = module.output_dtype()
        self._world_size = env.world_size
        self._device_type = (device.type if device is not None else ("cuda" if torch.cuda.is_available() else "cpu"))
        self._out_device = device if device is not None else _device_for(0, self._device_type)
        W = self._world_size
        tw: List[List[Any]] = [[] for _ in range(W)]
        rw: List[List[Any]] = [[] for _ in range(W)]
        cw: List[List[Any]] = [[] for _ in range(W)]
        slices: Dict[Any, torch.Tensor] = {}  # (kind, rank, table) -> packed rows of that shard
        self._rw_tables: List[Any] = []
        self._rw_mean_features: List[str] = []
        self._cw_order: Dict[str, List[int]] = {}  # table -> ranks in column order
        for cfg in self._configs:
            ps = table_name_to_parameter_sharding[cfg.name]
            packed = module.embedding_bags[cfg.name].weight
            bits = BITS[cfg.data_type]
            if ps.sharding_type == ShardingType.TABLE_WISE.value:
                tw[ps.ranks[0]].append(cfg)
                slices[("tw", ps.ranks[0], cfg.name)] = packed
            elif ps.sharding_type == ShardingType.ROW_WISE.value:
                block = (cfg.num_embeddings + W - 1) // W
                self._rw_tables.append((cfg, block))
                if cfg.pooling == PoolingType.MEAN:
                    self._rw_mean_features.extend(cfg.feature_names)
                for r in range(W):
                    rows = max(0, min(block, cfg.num_embeddings - r * block))
                    local = copy.deepcopy(cfg)
                    local.num_embeddings = max(rows, 1)  # an empty block keeps one unused row so the kernel has a table
                    local.pooling = PoolingType.SUM  # the divisor of a mean needs the whole bag: applied after the sum over devices
                    rw[r].append(local)
                    part = packed[r * block: r * block + rows]
                    slices[("rw", r, cfg.name)] = part if rows > 0 else packed.new_zeros(1, packed.shape[1])
            elif ps.sharding_type == ShardingType.COLUMN_WISE.value:
                ranks = list(ps.ranks)
                if len(set(ranks)) != len(ranks):
                    raise ValueError(f"column-wise shards of {cfg.name} must sit on distinct devices, got ranks {ranks}")
                if cfg.embedding_dim % len(ranks):
                    raise ValueError(f"{cfg.name}: embedding_dim {cfg.embedding_dim} is not divisible into {len(ranks)} column shards")
                width = cfg.embedding_dim // len(ranks)
                payload = cfg.embedding_dim * bits // 8
                self._cw_order[cfg.name] = ranks
                for j, r in enumerate(ranks):
                    local = copy.deepcopy(cfg)
                    local.embedding_dim = width
                    cw[r].append(local)
                    cols = packed[:, j * width * bits // 8: (j + 1) * width * bits // 8]
                    slices[("cw", r, cfg.name)] = torch.cat([cols, packed[:, payload:]], dim=1) if bits < 16 else cols
            else:
                raise ValueError(f"quantized inference sharding supports table_wise, row_wise and column_wise placement, got {ps.sharding_type} for {cfg.name}")

        def build(kind: str, per_rank: List[List[Any]]) -> nn.ModuleList:
            out = nn.ModuleList()
            for rank, cfgs in enumerate(per_rank):
                if not cfgs:
                    out.append(nn.Identity())
                    continue
                dev = _device_for(rank, self._device_type)
                shard = QuantEmbeddingBagCollection(copy.deepcopy(cfgs), self._is_weighted, dev, output_dtype=module.output_dtype())
                for cfg in cfgs:
                    piece = slices[(kind, rank, cfg.name)]
                    if not piece.is_meta:  # a module built on the meta device is sharded without data: the caller loads every shard in place
                        shard.embedding_bags[cfg.name].weight.copy_(piece.to(dev))
                out.append(shard)
            return out

        self._shards = build("tw", tw)
        self._rw_shards = build("rw", rw)
        self._cw_shards = build("cw", cw)
        self._feature_names_per_rank: List[List[str]] = [[f for c in cfgs for f in c.feature_names] for cfgs in tw]
        self._cw_feature_names_per_rank: List[List[str]] = [[f for c in cfgs for f in c.feature_names] for cfgs in cw]
        self._rw_feature_names: List[str] = [f for cfg, _ in self._rw_tables for f in cfg.feature_names]
        self.register_buffer("_rw_block_sizes", torch.tensor([b for cfg, b in self._rw_tables for _ in cfg.feature_names], dtype=torch.int64), persistent=False)
        # embedding name (feature, or feature@table when a feature feeds several tables) -> how its output is assembled
        self._embedding_names = module._embedding_names
        self._length_per_key = module._length_per_key
        self._name_kind: Dict[str, str] = {}
        self._name_table: Dict[str, str] = {}
        i = 0
        for cfg in self._configs:
            kind = {ShardingType.TABLE_WISE.value: "tw", ShardingType.ROW_WISE.value: "rw", ShardingType.COLUMN_WISE.value: "cw"}[table_name_to_parameter_sharding[cfg.name].sharding_type]
            for _ in cfg.feature_names:
                self._name_kind[self._embedding_names[i]] = kind
                self._name_table[self._embedding_names[i]] = cfg.name
                i += 1

        self._input_dist = ShardedQuantEbcInputDist(
            W, self._device_type, dict(enumerate(self._feature_names_per_rank)), dict(enumerate(self._cw_feature_names_per_rank)), {r: r for r in range(W)},
            self._rw_feature_names, self._rw_block_sizes)
        self._init_quant_state("embedding_bags", {c.name: table_name_to_parameter_sharding[c.name].sharding_type for c in self._configs})

    def _local(self, features: KeyedJaggedTensor, keys: List[str], names: List[str], rank: int) -> KeyedJaggedTensor:
        return features.permute([keys.index(f) for f in names]).to(_device_for(rank, self._device_type), non_blocking=True)

    def forward(self, features: KeyedJaggedTensor) -> KeyedTensor:
        keys = features.keys()
        if self._device_type == "cuda" and not self._rw_feature_names:
            return self._forward_direct(features, keys)
        dist = self._input_dist(features)
        pieces: Dict[str, torch.Tensor] = {}
        for rank, local in dist.table_wise.items():
            for k, v in self._shards[rank](local).to_dict().items():
                pieces[k] = v.to(self._out_device, non_blocking=True)
        for rank, local in enumerate(dist.row_wise):
            for k, v in self._rw_shards[rank](local).to_dict().items():
                v = v.to(self._out_device, non_blocking=True)
                pieces[k] = v if k not in pieces or rank == 0 else pieces[k] + v
        if dist.row_wise and self._rw_mean_features:
            lens = dist.row_wise_request.lengths().view(len(self._rw_feature_names), -1).to(self._out_device)
            for name in self._embedding_names:
                f = name.split("@")[0]
                if self._name_kind.get(name) == "rw" and f in self._rw_mean_features:
                    pieces[name] = pieces[name] / lens[self._rw_feature_names.index(f)].clamp(min=1).unsqueeze(1).to(pieces[name].dtype)
        cw_parts: Dict[str, Dict[int, torch.Tensor]] = {}
        for rank, local in dist.column_wise.items():
            for k, v in self._cw_shards[rank](local).to_dict().items():
                cw_parts.setdefault(k, {})[rank] = v.to(self._out_device, non_blocking=True)
        for name, by_rank in cw_parts.items():
            pieces[name] = torch.cat([by_rank[r] for r in self._cw_order[self._name_table[name]]], dim=1)
        values = torch.cat([pieces[n] for n in self._embedding_names], dim=1)
        return KeyedTensor(keys=self._embedding_names, values=values, length_per_key=self._length_per_key)

    def _forward_direct(self, features: KeyedJaggedTensor, keys: List[str]) -> KeyedTensor:
        """Table-wise and column-wise shards on GPUs: every device's lookup kernel stores its pooled rows straight into the
        result buffer on the output device, at the final column of each embedding (column shards at their offset inside it).
        No per-table copy, no concatenation; the output device's stream waits for one event per contributing device."""
        out_dev = self._out_device
        col, start = {}, 0
        for name, width in zip(self._embedding_names, self._length_per_key):
            col[name] = start
            start += width
        out = torch.empty((features.stride(), start), dtype=self._out_dtype, device=out_dev)
        out_stream = torch.cuda.current_stream(out_dev)
        ready = torch.cuda.Event()
        ready.record(out_stream)  # the buffer exists (allocator-wise) before a peer writes into it
        done = []
        for kind, shards, names_per_rank in (("tw", self._shards, self._feature_names_per_rank), ("cw", self._cw_shards, self._cw_feature_names_per_rank)):
            for rank, (shard, fnames) in enumerate(zip(shards, names_per_rank)):
                if not fnames:
                    continue
                dev = _device_for(rank, self._device_type)
                local = self._local(features, keys, fnames, rank)
                columns = dict(col)
                if kind == "cw":
                    for name in shard._embedding_names:
                        order = self._cw_order[self._name_table[name]]
                        columns[name] = col[name] + order.index(rank) * (self._length_per_key[self._embedding_names.index(name)] // len(order))
                with torch.cuda.device(dev):
                    stream = torch.cuda.current_stream(dev)
                    stream.wait_event(ready)
                    shard.forward_into(local, out, columns)
                    ev = torch.cuda.Event()
                    ev.record(stream)
                    done.append(ev)
        for ev in done:
            out_stream.wait_event(ev)
        return KeyedTensor(keys=self._embedding_names, values=out, length_per_key=self._length_per_key)

    def sharded_parameter_names(self, prefix: str = ""):
        for attr in ("_shards", "_rw_shards", "_cw_shards"):
            for rank, shard in enumerate(getattr(self, attr)):
                if isinstance(shard, QuantEmbeddingBagCollection):
                    for name in shard.embedding_bags.keys():
                        yield f"{prefix}{attr}.{rank}.embedding_bags.{name}.weight"


class QuantEmbeddingBagCollectionSharder(BaseQuantEmbeddingSharder[QuantEmbeddingBagCollection]):
    def shard(self, module: QuantEmbeddingBagCollection, params: Dict[str, ParameterSharding], env: ShardingEnv,
              device: Optional[torch.device] = None, module_fqn: Optional[str] = None) -> ShardedQuantEmbeddingBagCollection:
        return ShardedQuantEmbeddingBagCollection(module, params, env, getattr(self, "fused_params", None), device)

    def shardable_parameters(self, module: QuantEmbeddingBagCollection) -> Dict[str, torch.Tensor]:
        return {name: m.weight for name, m in module.embedding_bags.items()}

    def sharding_types(self, compute_device_type: str) -> List[str]:
        return [ShardingType.TABLE_WISE.value, ShardingType.ROW_WISE.value, ShardingType.COLUMN_WISE.value]

    @property
    def module_type(self) -> Type[QuantEmbeddingBagCollection]:
        return QuantEmbeddingBagCollection


class ShardedQuantFeatureProcessedEmbeddingBagCollection(ShardedQuantEmbeddingBagCollection):
    """Sharded form of the quantized feature-processed collection: the processors (position weights, a few KB) run once on
    the request before it is cut up for the devices; the per-id weights they produce travel with the ids
    (``torchrec/distributed/quant_embeddingbag.py:471-620``)."""

    def __init__(self, module: QuantFeatureProcessedEmbeddingBagCollection, table_name_to_parameter_sharding: Dict[str, ParameterSharding],
                 env: ShardingEnv, fused_params: Optional[Dict[str, Any]] = None, device: Optional[torch.device] = None) -> None:
        super().__init__(module, table_name_to_parameter_sharding, env, fused_params, device)
        self.feature_processor = copy.deepcopy(module.feature_processor)

    def forward(self, features: KeyedJaggedTensor) -> KeyedTensor:
        fp = self.feature_processor
        first = next(fp.parameters(), None)
        if first is not None and first.device != features.values().device:
            fp.to(features.values().device)
        return super().forward(fp(features))


class QuantFeatureProcessedEmbeddingBagCollectionSharder(BaseQuantEmbeddingSharder[QuantFeatureProcessedEmbeddingBagCollection]):
    def shard(self, module: QuantFeatureProcessedEmbeddingBagCollection, params: Dict[str, ParameterSharding], env: ShardingEnv,
              device: Optional[torch.device] = None, module_fqn: Optional[str] = None) -> ShardedQuantFeatureProcessedEmbeddingBagCollection:
        return ShardedQuantFeatureProcessedEmbeddingBagCollection(module, params, env, getattr(self, "fused_params", None), device)

    def shardable_parameters(self, module: QuantFeatureProcessedEmbeddingBagCollection) -> Dict[str, torch.Tensor]:
        return {name: m.weight for name, m in module.embedding_bags.items()}

    def sharding_types(self, compute_device_type: str) -> List[str]:
        return [ShardingType.TABLE_WISE.value, ShardingType.ROW_WISE.value, ShardingType.COLUMN_WISE.value]

    @property
    def module_type(self) -> Type[QuantFeatureProcessedEmbeddingBagCollection]:
        return QuantFeatureProcessedEmbeddingBagCollection
