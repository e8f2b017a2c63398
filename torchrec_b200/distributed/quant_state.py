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
