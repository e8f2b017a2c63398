"""In-training embedding pruning (ITEP): train a table of ``num_embeddings`` rows against an id space of ``unpruned`` ids.

State per pruned table (checkpointed as ``<table>_itp_address_lookup`` / ``<table>_itp_row_util``):

* ``address_lookup[unpruned]`` -- where an id reads: an entry ``v >= 0`` means the id *owns* row ``v``; ``v < 0`` means it shares row
  ``-(v+1)`` with that row's owner.  Initially the first ``num_embeddings`` ids own their row and the others share row
  ``id % num_embeddings``.
* ``row_util[unpruned]`` -- how often each id was seen (sampled on a fixed schedule, halved at every pruning).

Every step the ids of the pruned tables go through ``ops.sparse_ops.itep_remap`` (one kernel: remap + utilisation count).  On the
pruning schedule, rows move from the least used owners to the most used non-owners; a row that changes hands has its weights
re-initialised and its optimizer state zeroed.

Counterpart of ``torchrec/modules/itep_modules.py`` (``GenericITEPModule`` ``:38``, ``RowwiseShardedITEPModule`` ``:551``); the
reference keeps the same two buffers but leaves the remap and the pruning rule to operators of an external wheel.
"""
from __future__ import annotations

import logging
import math
from typing import Dict, List, Optional, Tuple, Type

import torch
import torch.distributed as dist
from torch import nn
from torch.nn.parallel import DistributedDataParallel

from torchrec_b200.modules.pruning_logger import PruningLogger, PruningLoggerDefault
from torchrec_b200.ops import sparse_ops as sops
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

logger: logging.Logger = logging.getLogger(__name__)


def init_address_lookup(address_lookup: torch.Tensor, buffer_offsets: List[int], emb_sizes: List[int]) -> None:
    """First ``emb_size`` ids of every buffer own their row, the rest share row ``id % emb_size``."""
    for b, size in enumerate(emb_sizes):
        lo, hi = buffer_offsets[b], buffer_offsets[b + 1]
        ids = torch.arange(hi - lo, dtype=torch.int64, device=address_lookup.device)
        address_lookup[lo:hi] = torch.where(ids < size, ids, -(ids % max(size, 1) + 1)) if size > 0 else -1


def prune_embedding_tables(address_lookup: torch.Tensor, row_util: torch.Tensor, buffer_offsets: List[int], emb_sizes: List[int],
                           decay: float = 0.5) -> Tuple[torch.Tensor, torch.Tensor]:
    """Hand rows from little-used owners to much-used sharers.  Returns ``(rows that changed owner, offsets per buffer)``."""
    pruned: List[torch.Tensor] = []
    offsets = [0]
    for b, size in enumerate(emb_sizes):
        lo, hi = buffer_offsets[b], buffer_offsets[b + 1]
        al, util = address_lookup[lo:hi], row_util[lo:hi]
        owners = (al >= 0).nonzero().view(-1)
        sharers = ((al < 0) & (util > 0)).nonzero().view(-1)
        n = min(owners.numel(), sharers.numel())
        moved = al.new_empty(0)
        if n > 0:
            o_util, o_order = util[owners].sort(stable=True)
            s_util, s_order = util[sharers].sort(descending=True, stable=True)
            swap = s_util[:n] > o_util[:n]  # a prefix: owners ascend, sharers descend
            k = int(swap.sum())
            if k > 0:
                losers, winners = owners[o_order[:k]], sharers[s_order[:k]]
                moved = al[losers].clone()
                al[winners] = moved
                al[losers] = -(losers % max(size, 1) + 1)
                # a loser that would share the row it just lost, or any row: its reads go to whoever owns that row now
        pruned.append(moved)
        offsets.append(offsets[-1] + moved.numel())
        util.mul_(decay)
    cat = torch.cat(pruned) if pruned else address_lookup.new_empty(0)
    return cat, torch.tensor(offsets, dtype=torch.int64)


class GenericITEPModule(nn.Module):
    """``forward(KJT, cur_iter) -> KJT`` with the ids of pruned tables remapped; tables held whole on this rank
    (table-wise / column-wise shards, or an unsharded collection passed as ``lookups=[ebc]``)."""

    def __init__(
        self,
        table_name_to_unpruned_hash_sizes: Dict[str, int],
        lookups: Optional[List[nn.Module]] = None,
        enable_pruning: bool = True,
        pruning_interval: int = 1001,
        pg: Optional[dist.ProcessGroup] = None,
        table_name_to_sharding_type: Optional[Dict[str, str]] = None,
        pruning_logger_type: Type[PruningLogger] = PruningLoggerDefault,
    ) -> None:
        super().__init__()
        self.pruning_logger = pruning_logger_type
        with self.pruning_logger.pruning_logger(event="ITEP_MODULE_INIT") as details:
            details.enable_pruning = enable_pruning
            details.pruning_interval = pruning_interval
            self.enable_pruning = enable_pruning
            self.pruning_interval = pruning_interval
            self.lookups: List[nn.Module] = list(lookups) if lookups else []
            self.table_name_to_unpruned_hash_sizes = table_name_to_unpruned_hash_sizes
            self.table_name_to_sharding_type = table_name_to_sharding_type or {}
            self.feature_table_map: Dict[str, int] = {}
            self.table_name_to_idx: Dict[str, int] = {}
            self.idx_to_table_name: Dict[int, str] = {}
            self.buffer_offsets_list: List[int] = [0]
            self.emb_sizes_list: List[int] = []
            self.last_pruned_iter = -1
            self.pg = pg
            self.current_device: Optional[torch.device] = None
            self._remap_cache: Dict[Tuple[str, ...], torch.Tensor] = {}
            if self.lookups:
                self.init_itep_state()

    # ---- tables --------------------------------------------------------------------------------------
    def _tables(self):
        """``(table config, weight getter, optimizer-state getter)`` of every table of the lookups, sharded or not."""
        for lookup in self.lookups:
            while isinstance(lookup, DistributedDataParallel):
                lookup = lookup.module
            if hasattr(lookup, "emb_modules"):
                for emb in lookup.emb_modules:
                    tbe = emb.emb_module
                    states = tbe.split_optimizer_states() if getattr(tbe, "fused", False) else [{} for _ in emb.config.embedding_tables]
                    for t, w, st in zip(emb.config.embedding_tables, emb.split_embedding_weights(), states):
                        yield t, w, st
            else:  # an unsharded EmbeddingBagCollection / EmbeddingCollection
                configs = lookup.embedding_bag_configs() if hasattr(lookup, "embedding_bag_configs") else lookup.embedding_configs()
                mods = lookup.embedding_bags if hasattr(lookup, "embedding_bags") else lookup.embeddings
                for c in configs:
                    yield c, mods[c.name].weight, {}

    def get_table_hash_sizes(self, table) -> Tuple[int, int]:
        """``(rows held here, unpruned ids routed here)`` of a table."""
        rows = getattr(table, "local_rows", None) or table.num_embeddings
        return rows, self.table_name_to_unpruned_hash_sizes.get(table.name, rows)

    def init_itep_state(self) -> None:
        names: List[str] = []
        for table, weight, _ in self._tables():
            if table.name in self.table_name_to_idx:
                continue
            pruned, unpruned = self.get_table_hash_sizes(table)
            if pruned == unpruned:
                continue
            assert unpruned > pruned, f"table {table.name}: unpruned size {unpruned} is smaller than its {pruned} rows"
            idx = len(names)
            names.append(table.name)
            self.buffer_offsets_list.append(self.buffer_offsets_list[-1] + unpruned)
            self.emb_sizes_list.append(pruned)
            for f in table.feature_names:
                self.feature_table_map[f] = idx
            self.table_name_to_idx[table.name] = idx
            self.idx_to_table_name[idx] = table.name
            dev = weight.device
            assert self.current_device is None or self.current_device == dev, "pruned tables of one module must share a device"
            self.current_device = dev
        if self.current_device is None:
            self.current_device = torch.device("cpu")
        self.create_itep_buffers(self.buffer_offsets_list[-1], self.buffer_offsets_list, names, self.emb_sizes_list)
        init_address_lookup(self.address_lookup, self.buffer_offsets_list, self.emb_sizes_list)

    def create_itep_buffers(self, buffer_size: int, buffer_offsets: List[int], table_names: List[str], emb_sizes: List[int]) -> None:
        """One flat pair of buffers; every table's slice is registered under its own name so it is checkpointed per table."""
        dev = self.current_device
        self.buffer_offsets = torch.tensor(buffer_offsets, dtype=torch.int64, device=dev)
        self.emb_sizes = torch.tensor(emb_sizes, dtype=torch.int64, device=dev)
        self.address_lookup = torch.zeros(buffer_size, dtype=torch.int64, device=dev)
        self.row_util = torch.zeros(buffer_size, dtype=torch.float32, device=dev)
        for i, name in enumerate(table_names):
            self.register_buffer(f"{name}_itp_address_lookup", self.address_lookup[buffer_offsets[i]:buffer_offsets[i + 1]])
            self.register_buffer(f"{name}_itp_row_util", self.row_util[buffer_offsets[i]:buffer_offsets[i + 1]])

    # ---- pruning -------------------------------------------------------------------------------------
    @torch.no_grad()
    def reset_weight_momentum(self, pruned_indices: torch.Tensor, pruned_indices_offsets: torch.Tensor) -> None:
        offs = pruned_indices_offsets.tolist()
        done = set()
        for table, weight, states in self._tables():
            idx = self.table_name_to_idx.get(table.name)
            if idx is None or offs[idx + 1] == offs[idx]:
                continue
            rows = pruned_indices[offs[idx]:offs[idx + 1]].to(weight.device)
            rows = rows[rows < weight.shape[0]]
            bound = math.sqrt(1.0 / max(table.num_embeddings, 1))
            weight[rows] = torch.empty(rows.numel(), weight.shape[1], device=weight.device).uniform_(-bound, bound).to(weight.dtype)
            for s in states.values():
                if s.dim() >= 1 and s.shape[0] >= weight.shape[0]:
                    s[rows] = 0
            done.add(table.name)

    def flush_uvm_cache(self) -> None:
        for lookup in self.lookups:
            while isinstance(lookup, DistributedDataParallel):
                lookup = lookup.module
            if hasattr(lookup, "flush"):
                lookup.flush()

    def print_itep_eviction_stats(self, pruned_indices_offsets: torch.Tensor, pruned_indices_total_length: int, cur_iter: int) -> None:
        offs = pruned_indices_offsets.tolist()
        for idx, name in self.idx_to_table_name.items():
            n, size = offs[idx + 1] - offs[idx], self.emb_sizes_list[idx]
            logger.info("ITEP iter %d: table %s handed over %d of %d rows (%.2f%%)", cur_iter, name, n, size, 100.0 * n / max(size, 1))

    @staticmethod
    def _start_pruning(cur_iter: int, interval: int) -> bool:
        return ((cur_iter < 10 and (cur_iter + 1) % 3 == 0) or (cur_iter < 100 and (cur_iter + 1) % 30 == 0)
                or (cur_iter < 1000 and (cur_iter + 1) % 300 == 0) or ((cur_iter + 1) % interval == 0))

    @staticmethod
    def _update_util(cur_iter: int) -> bool:
        return cur_iter < 10 or (cur_iter < 100 and (cur_iter + 1) % 19 == 0) or ((cur_iter + 1) % 39 == 0)

    def _feature_buffer(self, keys: List[str], device: torch.device) -> torch.Tensor:
        k = tuple(keys)
        t = self._remap_cache.get(k)
        if t is None or t.device != device:
            t = torch.tensor([self.feature_table_map.get(f, -1) for f in keys], dtype=torch.int32, device=device)
            self._remap_cache[k] = t
        return t

    def forward(self, sparse_features: KeyedJaggedTensor, cur_iter: int) -> KeyedJaggedTensor:
        if not self.enable_pruning or not self.lookups or len(self.emb_sizes_list) == 0:
            return sparse_features
        cur_iter = int(cur_iter)
        if self.training and self._start_pruning(cur_iter, self.pruning_interval) and self.last_pruned_iter != cur_iter:
            pruned, offsets = prune_embedding_tables(self.address_lookup, self.row_util, self.buffer_offsets_list, self.emb_sizes_list)
            if pruned.numel() > 0:
                self.reset_weight_momentum(pruned, offsets)
                self.flush_uvm_cache()
            self.last_pruned_iter = cur_iter
            self.print_itep_eviction_stats(offsets, int(pruned.numel()), cur_iter)
        keys = sparse_features.keys()
        values = sparse_features.values()
        if values.numel() == 0 or not any(k in self.feature_table_map for k in keys):
            return sparse_features
        if sparse_features.variable_stride_per_key():
            lpk = torch.tensor([0] + sparse_features.length_per_key(), dtype=torch.int64).cumsum(0)
            feature_offsets = lpk.to(values.device)
        else:
            B = sparse_features.stride()
            feature_offsets = sparse_features.offsets()[:: max(B, 1)] if B > 0 else torch.zeros(len(keys) + 1, dtype=torch.int64, device=values.device)
        remapped = sops.itep_remap(values, feature_offsets, self._feature_buffer(keys, values.device), self.address_lookup, self.row_util, self.buffer_offsets,
                                   update_util=self.training and self._update_util(cur_iter))
        return KeyedJaggedTensor(
            keys=keys, values=remapped, weights=sparse_features.weights_or_none(), lengths=sparse_features.lengths(), offsets=sparse_features.offsets(),
            stride=sparse_features.stride() if not sparse_features.variable_stride_per_key() else None,
            stride_per_key_per_rank=sparse_features.stride_per_key_per_rank() if sparse_features.variable_stride_per_key() else None,
            inverse_indices=sparse_features.inverse_indices_or_none())


class RowwiseShardedITEPModule(GenericITEPModule):
    """Row-wise (and table-row-wise) shards: the input distribution cuts the *unpruned* id space into equal blocks, so this
    rank receives ids ``[0, block)`` of its block and maps them onto its ``local_rows`` rows."""

    def _get_local_unpruned_hash_sizes_and_offsets(self, table, sharding_type: str) -> Tuple[List[int], List[int]]:
        shards = table.global_metadata.shards_metadata
        n = len(shards)
        total = self.table_name_to_unpruned_hash_sizes[table.name]
        block = math.ceil(total / n)
        sizes = [max(0, min(block, total - r * block)) for r in range(n)]
        offsets = [0]
        for s in sizes[:-1]:
            offsets.append(offsets[-1] + s)
        return sizes, offsets

    def get_table_hash_sizes(self, table) -> Tuple[int, int]:
        rows = table.local_rows
        if table.name not in self.table_name_to_unpruned_hash_sizes:
            return rows, rows
        sizes, _ = self._get_local_unpruned_hash_sizes_and_offsets(table, self.table_name_to_sharding_type.get(table.name, ""))
        shards = table.global_metadata.shards_metadata
        mine = next(i for i, s in enumerate(shards) if s == table.local_metadata)
        return rows, sizes[mine]
