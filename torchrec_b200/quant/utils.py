"""Helpers for quantized modules ahead of tracing and packaging: stable fx names for batched lookup kernels that are not
registered as named submodules, and replacing meta-device quantized collections with CPU ones.
Counterpart of ``torchrec/quant/utils.py:23-120``."""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from torchrec_b200.quant.embedding_modules import (
    MODULE_ATTR_REGISTER_TBES_BOOL,
    MODULE_ATTR_ROW_ALIGNMENT_INT,
    DEFAULT_ROW_ALIGNMENT,
    EmbeddingBagCollection as QuantEmbeddingBagCollection,
    EmbeddingCollection as QuantEmbeddingCollection,
)


def populate_fx_names(quant_ebc: nn.Module) -> None:
    """Give every batched kernel of a quantized (or sharded quantized) bag collection an ``_fx_path``: the tracer falls back to
    that name for modules it cannot find in ``named_modules``.  Unsharded: ``emb_module.<t1,t2,..>``.  Sharded: one
    ``embedding_lookup.rank_<r>`` per device shard and ``embedding_lookup.rank_<r>.group_<g>.tbe`` per kernel."""
    from torchrec_b200.distributed.quant_embeddingbag import ShardedQuantEmbeddingBagCollection

    if isinstance(quant_ebc, QuantEmbeddingBagCollection):
        for group, emb in zip(quant_ebc._group_tables, quant_ebc._emb_modules):
            emb._fx_path = "emb_module." + ",".join(t.name for t in group)
    elif isinstance(quant_ebc, ShardedQuantEmbeddingBagCollection):
        for rank, shard in enumerate(quant_ebc._shards):
            shard._fx_path = f"embedding_lookup.rank_{rank}"
            if isinstance(shard, QuantEmbeddingBagCollection):
                for g, emb in enumerate(shard._emb_modules):
                    emb._fx_path = f"embedding_lookup.rank_{rank}.group_{g}.tbe"


def recursive_populate_fx_names(module: nn.Module) -> None:
    from torchrec_b200.distributed.quant_embeddingbag import ShardedQuantEmbeddingBagCollection

    if isinstance(module, (QuantEmbeddingBagCollection, ShardedQuantEmbeddingBagCollection)):
        populate_fx_names(module)
        return
    for child in module.children():
        recursive_populate_fx_names(child)


def _was_built_on_meta(module: nn.Module) -> bool:
    dev = getattr(module, "_device", None)
    return dev is not None and torch.device(dev).type == "meta"


def meta_to_cpu_placement(module: nn.Module) -> None:
    """Swap every quantized collection that was constructed for the meta device (a placeholder left unsharded by the plan) for an
    equal collection on CPU, in place.  A ``DistributedModelParallel`` is read through ``.module`` and written through its wrapped
    attribute."""
    if hasattr(module, "_dmp_wrapped_module"):
        _meta_to_cpu_placement(module.module, module, "_dmp_wrapped_module")
    else:
        _meta_to_cpu_placement(module, module)


def _meta_to_cpu_placement(module: nn.Module, parent: nn.Module, name: Optional[str] = None) -> None:
    if name is not None and _was_built_on_meta(module) and isinstance(module, (QuantEmbeddingBagCollection, QuantEmbeddingCollection)):
        common = dict(device=torch.device("cpu"), output_dtype=module.output_dtype(),
                      register_tbes=getattr(module, MODULE_ATTR_REGISTER_TBES_BOOL, False),
                      row_alignment=getattr(module, MODULE_ATTR_ROW_ALIGNMENT_INT, DEFAULT_ROW_ALIGNMENT))
        if isinstance(module, QuantEmbeddingBagCollection):
            new = QuantEmbeddingBagCollection(tables=module.embedding_bag_configs(), is_weighted=module.is_weighted(), **common)
        else:
            new = QuantEmbeddingCollection(tables=module.embedding_configs(), need_indices=module.need_indices(), **common)
        setattr(parent, name, new)
        return
    for child_name, child in module.named_children():
        _meta_to_cpu_placement(child, module, child_name)
