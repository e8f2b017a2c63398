"""Dynamic resharding: change the placement of embedding tables of a live sharded module.

Every rank knows the old and the new shard layout of every table.  For each pair (old shard, new shard) whose row /
column ranges intersect, the owner of the old shard sends exactly the intersection to the owner of the new shard; all
sends and receives of a module are posted together as one batch of point-to-point operations (same order on every
rank), local intersections are plain copies.  Weights and fused-optimizer states (row-wise or element-wise) move the same
way, so training continues with identical numerics after the move.

Counterpart of ``torchrec/distributed/sharding/dynamic_sharding.py`` (``shards_all_to_all`` / ``transfer_data``
``:807-830``, optimizer state move ``update_optimizer_state_post_resharding``).
"""
from __future__ import annotations

import copy
import os
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import nn

from torchrec_b200.distributed.types import ParameterSharding, ShardedTensor


def _rank_of(placement) -> int:
    if hasattr(placement, "rank"):
        return int(placement.rank())
    s = str(placement)  # "rank:3/cuda:3"
    return int(s.split("/")[0].split(":")[1])


def _intersect(a_off: List[int], a_size: List[int], b_off: List[int], b_size: List[int]) -> Optional[Tuple[List[int], List[int]]]:
    off, size = [], []
    for ao, asz, bo, bsz in zip(a_off, a_size, b_off, b_size):
        lo, hi = max(ao, bo), min(ao + asz, bo + bsz)
        if hi <= lo:
            return None
        off.append(lo)
        size.append(hi - lo)
    return off, size


def _region(t: torch.Tensor, shard_off: List[int], off: List[int], size: List[int]) -> torch.Tensor:
    view = t
    for d, (so, o, n) in enumerate(zip(shard_off, off, size)):
        view = view.narrow(d, o - so, n)
    return view


def transfer_sharded_tensor(old_meta: List[Any], old_local: Dict[Tuple[int, ...], torch.Tensor], new_meta: List[Any], new_local: Dict[Tuple[int, ...], torch.Tensor],
                            pg: Optional[dist.ProcessGroup], ops: List[Any], post: List[Any]) -> None:
    """Queue the transfers that fill the new local shards from the old layout.  ``old_meta`` / ``new_meta``: shard metadata
    (offsets, sizes, placement) of the whole tensor; ``*_local``: this rank's shard tensors keyed by their offsets.
    Point-to-point ops are appended to ``ops``; copies to run after they complete to ``post``."""
    rank = dist.get_rank(pg) if pg is not None else 0
    for o in old_meta:
        o_rank, o_off, o_size = _rank_of(o.placement), list(o.shard_offsets), list(o.shard_sizes)
        for n in new_meta:
            n_rank, n_off, n_size = _rank_of(n.placement), list(n.shard_offsets), list(n.shard_sizes)
            inter = _intersect(o_off, o_size, n_off, n_size)
            if inter is None:
                continue
            off, size = inter
            if rank == o_rank and rank == n_rank:
                src = _region(old_local[tuple(o_off)], o_off, off, size)
                dst = _region(new_local[tuple(n_off)], n_off, off, size)
                post.append((dst, src.detach().clone()))
            elif rank == o_rank:
                buf = _region(old_local[tuple(o_off)], o_off, off, size).detach().contiguous()
                ops.append(dist.P2POp(dist.isend, buf, dist.get_global_rank(pg, n_rank) if pg is not None else n_rank, group=pg))
            elif rank == n_rank:
                dst = _region(new_local[tuple(n_off)], n_off, off, size)
                buf = torch.empty(size, dtype=dst.dtype, device=dst.device)
                ops.append(dist.P2POp(dist.irecv, buf, dist.get_global_rank(pg, o_rank) if pg is not None else o_rank, group=pg))
                post.append((dst, buf))


class _RowShard:
    """Row range of a shard, with the placement of the shard that holds column 0 of those rows."""

    def __init__(self, off: int, size: int, placement: Any) -> None:
        self.shard_offsets, self.shard_sizes, self.placement = [off], [size], placement


def _row_meta(shards: List[Any]) -> List[_RowShard]:
    return [_RowShard(s.shard_offsets[0], s.shard_sizes[0], s.placement) for s in shards if s.shard_offsets[1] == 0]


def _is_rowwise(o_s, n_s, table: str, name: str) -> bool:
    for d in (o_s, n_s):
        for t in d.get(table, {}).get(name, {}).values():
            return t.dim() == 1
    return False


def _local_tensors(module: nn.Module) -> Tuple[Dict[str, Dict[Tuple[int, ...], torch.Tensor]], Dict[str, Dict[str, Dict[Tuple[int, ...], torch.Tensor]]]]:
    """This rank's weight and optimizer-state views of every table, keyed by the shard's (row, column) offsets."""
    from torch.nn.parallel import DistributedDataParallel

    weights: Dict[str, Dict[Tuple[int, ...], torch.Tensor]] = {}
    states: Dict[str, Dict[str, Dict[Tuple[int, ...], torch.Tensor]]] = {}
    for lookup in module._lookups:
        lk = lookup.module if isinstance(lookup, DistributedDataParallel) else lookup
        for emb in getattr(lk, "emb_modules", []):
            tbe = emb.emb_module
            split_states = tbe.split_optimizer_states() if getattr(tbe, "fused", False) else [{} for _ in emb.config.embedding_tables]
            for t, w, st in zip(emb.config.embedding_tables, emb.split_embedding_weights(), split_states):
                if t.local_metadata is None:
                    continue
                key = tuple(t.local_metadata.shard_offsets)
                weights.setdefault(t.name, {})[key] = w
                for sname, v in st.items():
                    states.setdefault(t.name, {}).setdefault(sname, {})[key] = v
    return weights, states


def _local_shards_by_offset(st: Any) -> Dict[Tuple[int, ...], torch.Tensor]:
    return {tuple(s.metadata.shard_offsets): s.tensor for s in st.local_shards()} if st is not None else {}


def _flush(ops: List[Any], post: List[Any]) -> None:
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()
    with torch.no_grad():
        for dst, src in post:
            dst.copy_(src)


def reshard_module(dmp: nn.Module, sharded_module_fqn: str, sharded_module: nn.Module, changed_shard_to_params: Dict[str, ParameterSharding]) -> nn.Module:
    """Build the module again under the new plan, move weights and optimizer states, and put it in place of the old one."""
    from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection

    old = sharded_module
    pg = old._env.process_group
    new_plan = copy.deepcopy(dict(old.module_sharding_plan))
    for table, ps in changed_shard_to_params.items():
        assert table in new_plan, f"{table} is not a table of {sharded_module_fqn}"
        new_plan[table] = ps
    # optimizer and kernel settings travel as fused params (every table of the module shares them)
    fused_params: Dict[str, Any] = {}
    for infos in old.sharding_type_to_sharding_infos.values():
        for info in infos:
            fused_params = dict(info.fused_params or {})
            break
        if fused_params:
            break
    for k in ("cache_load_factor", "enforce_hbm", "stochastic_rounding", "bounds_check_mode", "output_dtype_override"):
        fused_params.pop(k, None)
    stub = EmbeddingBagCollection(tables=copy.deepcopy(old._embedding_bag_configs), is_weighted=old._is_weighted, device=torch.device("meta"))
    new = type(old)(module=stub, table_name_to_parameter_sharding=new_plan, env=old._env, fused_params=fused_params, device=old._device,
                    qcomm_codecs_registry=old.qcomm_codecs_registry, module_fqn=sharded_module_fqn)
    ops: List[Any] = []
    post: List[Any] = []
    attr = old._TABLE_ATTR
    o_w, o_s = _local_tensors(old)
    n_w, n_s = _local_tensors(new)
    old_plan = old.module_sharding_plan
    for table in new_plan.keys():
        o_spec, n_spec = old_plan[table].sharding_spec, new_plan[table].sharding_spec
        if o_spec is None or n_spec is None:
            # data-parallel on one side: every rank holds the whole table
            if o_spec is None and n_spec is None:
                post.append((getattr(new, attr)[table].weight.detach(), getattr(old, attr)[table].weight.detach().clone()))
            continue
        transfer_sharded_tensor(o_spec.shards, o_w.get(table, {}), n_spec.shards, n_w.get(table, {}), pg, ops, post)
        # optimizer states: element-wise states are laid out like the weights, row-wise ones like their rows (the shard at
        # column 0 of every row block carries them)
        names = set()
        for d in (o_s.get(table, {}), n_s.get(table, {})):
            names.update(d.keys())
        # ranks without a local shard do not know the state names: agree on them
        gathered: List[Any] = [None] * dist.get_world_size(pg)
        dist.all_gather_object(gathered, sorted((n, _is_rowwise(o_s, n_s, table, n)) for n in names), group=pg)
        rowwise_of: Dict[str, bool] = {}
        for g in gathered:
            for n, rw in g:
                rowwise_of[n] = rowwise_of.get(n, False) or bool(rw)
        for sname, rowwise in sorted(rowwise_of.items()):
            if rowwise:
                o_meta, n_meta = _row_meta(o_spec.shards), _row_meta(n_spec.shards)
                o_loc = {(k[0],): v for k, v in o_s.get(table, {}).get(sname, {}).items() if k[1] == 0}
                n_loc = {(k[0],): v for k, v in n_s.get(table, {}).get(sname, {}).items() if k[1] == 0}
                transfer_sharded_tensor(o_meta, o_loc, n_meta, n_loc, pg, ops, post)
                # replicas of the row state on the other column shards of the same rows are refreshed locally afterwards
                for k, v in n_s.get(table, {}).get(sname, {}).items():
                    if k[1] != 0 and (k[0],) in n_loc:
                        post.append((v, n_loc[(k[0],)]))
            else:
                transfer_sharded_tensor(o_spec.shards, o_s.get(table, {}).get(sname, {}), n_spec.shards, n_s.get(table, {}).get(sname, {}), pg, ops, post)
    _flush(ops, post)
    # step counters of the kernels (bias correction) continue
    steps = [m.step for m in old.modules() if hasattr(m, "optimizer_args") and hasattr(m, "step") and isinstance(getattr(m, "step"), int)]
    for m in new.modules():
        if hasattr(m, "optimizer_args") and isinstance(getattr(m, "step", None), int) and steps:
            m.step = max(steps)
    parent = dmp.module
    parts = sharded_module_fqn.split(".")
    for p in parts[:-1]:
        parent = getattr(parent, p)
    setattr(parent, parts[-1], new)
    return new


# ---- helpers around a resharding call ---------------------------------------------------------------------
def update_module_sharding_plan(module: Any, changed_sharding_params: Dict[str, ParameterSharding],
                                sharding_type_to_sharding_infos: Dict[str, List[Any]]) -> None:
    """Write the new ``ParameterSharding`` of every changed table into the module's plan and into the sharding info that describes
    the table (looked up under the NEW sharding type: a table keeps its sharding type when it moves).
    Counterpart of ``torchrec/distributed/sharding/dynamic_sharding.py:835-869``."""
    if not hasattr(module, "module_sharding_plan"):
        raise RuntimeError("Module does not have a module_sharding_plan attribute")
    plan = module.module_sharding_plan
    for name, param in changed_sharding_params.items():
        plan[name] = param
        for info in sharding_type_to_sharding_infos.get(param.sharding_type, []):
            if info.embedding_config.name == name:
                info.param_sharding = param


def output_sharding_plan_delta_single(old_plan: Dict[str, ParameterSharding], new_plan: Dict[str, ParameterSharding],
                                      return_data_volume: bool = False) -> Tuple[float, Dict[str, ParameterSharding]]:
    """The tables of one module whose ranks differ between two plans, as the (copied) entries of the new plan - what
    ``DistributedModelParallel.reshard`` takes - and, on request, the MiB of fp32 weights those tables hold (else 0).  Both plans
    must name the same tables."""
    from torchrec_b200.distributed.types import EmbeddingModuleShardingPlan

    assert len(old_plan) == len(new_plan), "old and new plan must cover the same tables"
    diff = EmbeddingModuleShardingPlan({k: copy.deepcopy(v) for k, v in new_plan.items() if v.ranks != old_plan[k].ranks})
    volume = 0.0
    if return_data_volume:
        for sharding in diff.values():
            if sharding.sharding_spec is None:
                continue
            for shard in sharding.sharding_spec.shards:
                volume += shard.shard_sizes[0] * shard.shard_sizes[1] * 4 / (1024 * 1024)
    return volume, diff


def output_sharding_plans_delta(old_plan: Dict[str, Dict[str, ParameterSharding]], new_plan: Dict[str, Dict[str, ParameterSharding]],
                                return_data_volume: bool = False) -> Dict[str, Tuple[float, Dict[str, ParameterSharding]]]:
    """``output_sharding_plan_delta_single`` for every module of a whole-model plan (``ShardingPlan.plan``)."""
    out: Dict[str, Tuple[float, Dict[str, ParameterSharding]]] = {}
    for fqn, plan in old_plan.items():
        assert fqn in new_plan, f"Found mismatch between old and new plans, key: {fqn} not found in new plan"
        out[fqn] = output_sharding_plan_delta_single(plan, new_plan[fqn], return_data_volume)
    return out


def move_sharded_tensors_to_cpu(state_dict: Dict[str, Any]) -> Dict[str, Any]:
    """Move the local shards of every ``ShardedTensor`` inside a (nested) state dict to host memory, in place, and return the
    dict; other values are untouched.  Keeps a checkpoint-sized copy out of HBM while a resharding rebuilds the module."""

    def walk(item: Any) -> Any:
        if isinstance(item, ShardedTensor):
            for shard in item.local_shards():
                if shard.tensor.device.type != "cpu":
                    shard.tensor = shard.tensor.cpu()
            return item
        if isinstance(item, dict):
            return {k: walk(v) for k, v in item.items()}
        if isinstance(item, list):
            return [walk(v) for v in item]
        if isinstance(item, tuple):
            return tuple(walk(v) for v in item)
        return item

    out = walk(state_dict)
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
    return out
