"""Weight specs of a sharded quantized model: for every table shard inside every batched lookup kernel, which slice of which
unsharded tensor it holds.  Model publishing uses the map to cut an unsharded quantized checkpoint into per-device pieces.

Keys are ``<module path>.tbes.<kernel index>.<slot in kernel>.<table>.weight`` plus ``_qscale`` / ``_qbias`` for sub-16-bit tables
(payload bytes and the two fp16 row parameters are reported separately); values name the unsharded tensor, the shard's offsets
and sizes (column offsets and widths in payload bytes), and the sharding type.  Kernels are numbered over the table-wise
shards by device, then the row-wise shards, then the column-wise shards.  Counterpart of ``torchrec/distributed/quant_state.py:383-520``."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from torchrec_b200.distributed.types import ShardingType
from torchrec_b200.ops.quant_ops import BITS


@dataclass
class WeightSpec:
    fqn: str  # e.g. "ebc.embedding_bags.table_0.weight"
    shard_offsets: List[int]
    shard_sizes: List[int]
    sharding_type: Optional[str]
    virtual_table_dim_offsets: Optional[List[int]] = None


def get_param_id_from_type(is_sqebc: bool, is_sqmcec: bool, is_sfpebc: bool) -> str:
    """State-dict container of the tables for each kind of sharded quantized module."""
    if is_sqebc:
        return "embedding_bags"
    if is_sqmcec:
        return "_embedding_module.embeddings"
    if is_sfpebc:
        return "_embedding_bag_collection.embedding_bags"
    return "embeddings"


class ShardedQuantEmbeddingModuleState:
    """Checkpoint view of a sharded quantized collection under the UNSHARDED module's keys: ``<container>.<table>.weight`` is the
    packed table itself when it sits whole on one device, else a ``ShardedTensorBase`` whose local shards are the per-device
    pieces with their (row, payload-byte column) offsets; sub-16-bit tables also expose ``weight_qscalebias`` (the two fp16
    row parameters).  A publishing tool can thus read or overwrite a sharded serving model table by table without knowing where the
    pieces live.  The module provides ``_configs``, ``_shards`` / ``_rw_shards`` / ``_cw_shards`` and the row-block / column-order
    tables filled in by its constructor (``torchrec/distributed/quant_state.py:70-380``)."""

    def _init_quant_state(self, container: str, sharding_type_by_table: Dict[str, str]) -> None:
        self._state_container = container
        self._state_sharding = dict(sharding_type_by_table)

    def _pieces_of(self, table: str):
        """(row offset, payload column offset, packed rows) of every device's piece of ``table``."""
        kind = self._state_sharding[table]
        full = {c.name: c for c in self._configs}[table]
        bits = BITS[full.data_type]
        if kind == ShardingType.TABLE_WISE.value:
            for shard in self._shards:
                if hasattr(shard, self._state_container) and table in getattr(shard, self._state_container):
                    yield 0, 0, getattr(shard, self._state_container)[table].weight
        elif kind == ShardingType.ROW_WISE.value:
            block = {c.name: b for c, b in self._rw_tables}[table]
            for rank, shard in enumerate(self._rw_shards):
                rows = max(0, min(block, full.num_embeddings - rank * block))
                if rows > 0 and hasattr(shard, self._state_container):
                    yield rank * block, 0, getattr(shard, self._state_container)[table].weight[:rows]
        else:
            shards = self._cw_shards
            by_rank = dict(enumerate(shards)) if not isinstance(shards, torch.nn.ModuleDict) else None
            order = self._cw_order[table] if hasattr(self, "_cw_order") else next(r for c, r, _ in self._cw_tables if c.name == table)
            width_bytes = full.embedding_dim // len(order) * bits // 8
            for j, rank in enumerate(order):
                if by_rank is not None:
                    shard = by_rank[rank]
                else:
                    shard = shards[f"{rank}_{full.embedding_dim // len(order)}"]
                yield 0, j * width_bytes, getattr(shard, self._state_container)[table].weight

    def sharded_state_dict(self, prefix: str = "") -> Dict[str, object]:
        from torch.distributed._shard.sharded_tensor import Shard, ShardedTensorBase, ShardedTensorMetadata, ShardMetadata
        from torch.distributed._shard.sharded_tensor.metadata import TensorProperties

        out: Dict[str, object] = {}
        for cfg in self._configs:
            bits = BITS[cfg.data_type]
            payload = cfg.embedding_dim * bits // 8
            pieces = list(self._pieces_of(cfg.name))
            key = f"{prefix}{self._state_container}.{cfg.name}.weight"
            if self._state_sharding[cfg.name] == ShardingType.TABLE_WISE.value:
                whole = pieces[0][2]
                out[key] = whole[:, :payload] if bits < 16 else whole
                if bits < 16:
                    out[key + "_qscalebias"] = whole[:, payload: payload + 4]
                continue
            shards, tails = [], []
            for row_off, col_off, packed in pieces:
                width = packed.shape[1] - (4 if bits < 16 else 0)
                meta = ShardMetadata(shard_offsets=[row_off, col_off], shard_sizes=[packed.shape[0], width], placement=f"rank:0/{packed.device}")
                shards.append(Shard(tensor=packed[:, :width], metadata=meta))
                if bits < 16:
                    tails.append(Shard(tensor=packed[:, width: width + 4],
                                       metadata=ShardMetadata(shard_offsets=[row_off, 4 * (col_off // max(width, 1))], shard_sizes=[packed.shape[0], 4], placement=f"rank:0/{packed.device}")))

            def wrap(parts, size):
                props = TensorProperties(dtype=parts[0].tensor.dtype)
                meta = ShardedTensorMetadata(shards_metadata=[p.metadata for p in parts], size=torch.Size(size), tensor_properties=props)
                return ShardedTensorBase._init_from_local_shards_and_global_metadata(parts, meta)

            out[key] = wrap(shards, [cfg.num_embeddings, payload])
            if tails:
                n_col = len({p.metadata.shard_offsets[1] for p in tails})
                out[key + "_qscalebias"] = wrap(tails, [cfg.num_embeddings, 4 * n_col])
        return out


def sharded_tbes_weights_spec(sharded_model: torch.nn.Module, virtual_table_name_to_bucket_lengths: Optional[Dict[str, List[int]]] = None) -> Dict[str, WeightSpec]:
    """Walk ``sharded_model`` for sharded quantized collections and describe every table shard of every kernel."""
    from torchrec_b200.distributed.quant_embedding import ShardedQuantEmbeddingCollection
    from torchrec_b200.distributed.quant_embeddingbag import ShardedQuantEmbeddingBagCollection

    out: Dict[str, WeightSpec] = {}
    for module_fqn, module in sharded_model.named_modules():
        if not isinstance(module, (ShardedQuantEmbeddingBagCollection, ShardedQuantEmbeddingCollection)):
            continue
        container = get_param_id_from_type(isinstance(module, ShardedQuantEmbeddingBagCollection), False, False)
        prefix = f"{module_fqn}." if module_fqn else ""
        kernel = 0
        rw_block = {cfg.name: block for cfg, block in getattr(module, "_rw_tables", [])}
        full = {cfg.name: cfg for cfg in module._configs}
        if isinstance(module, ShardedQuantEmbeddingBagCollection):
            cw_ranks = dict(module._cw_order)
            cw_shards = [(r, s) for r, s in enumerate(module._cw_shards)]
        else:
            cw_ranks = {cfg.name: ranks for cfg, ranks, _ in module._cw_tables}
            cw_shards = [(int(key.split("_")[0]), s) for key, s in module._cw_shards.items()]
        groups = [("tw", r, s) for r, s in enumerate(module._shards)] + [("rw", r, s) for r, s in enumerate(module._rw_shards)] + [("cw", r, s) for r, s in cw_shards]
        for kind, rank, shard in groups:
            if not hasattr(shard, "_group_tables"):
                continue
            for group in shard._group_tables:
                for slot, table in enumerate(group):
                    bits = BITS[table.data_type]
                    rows = table.num_embeddings
                    payload = table.embedding_dim * bits // 8
                    row_off, col_off, stype = 0, 0, ShardingType.TABLE_WISE.value
                    if kind == "rw":
                        row_off, stype = rank * rw_block[table.name], ShardingType.ROW_WISE.value
                        rows = max(0, min(rw_block[table.name], full[table.name].num_embeddings - row_off))
                    elif kind == "cw":
                        col_off, stype = cw_ranks[table.name].index(rank) * payload, ShardingType.COLUMN_WISE.value
                    unsharded = f"{prefix}{container}.{table.name}.weight"
                    key = f"{prefix}tbes.{kernel}.{slot}.{table.name}.weight"
                    out[key] = WeightSpec(unsharded, [row_off, col_off], [rows, payload], stype)
                    if bits < 16:
                        for suffix in ("_qscale", "_qbias"):
                            out[key + suffix] = WeightSpec(unsharded + suffix, [row_off, 0], [rows, 2], stype)
                kernel += 1
    return out
