"""``EmbeddingShardingPlanner``: reserve -> enumerate -> (propose -> partition -> rate)* -> best plan.

``collective_plan`` runs the search on rank 0 and broadcasts the result so that every rank uses the
same plan.  Counterpart of ``torchrec/distributed/planner/planners.py:343-708``.
"""
from __future__ import annotations

import copy
import logging
import time
from functools import reduce
from typing import Callable, Dict, List, Optional, Tuple, Union, cast

import torch
import torch.distributed as dist
from torch import nn

from torchrec_b200.distributed.collective_utils import invoke_on_rank_and_broadcast_result
from torchrec_b200.distributed.comm import get_local_size
from torchrec_b200.distributed.planner.constants import BATCH_SIZE, MAX_SIZE
from torchrec_b200.distributed.planner.enumerators import EmbeddingEnumerator
from torchrec_b200.distributed.planner.partitioners import GreedyPerfPartitioner, MemoryBalancedPartitioner
from torchrec_b200.distributed.planner.perf_models import NoopPerfModel
from torchrec_b200.distributed.planner.proposers import GreedyProposer, GridSearchProposer, UniformProposer
from torchrec_b200.distributed.planner.storage_reservations import HeuristicalStorageReservation
from torchrec_b200.distributed.planner.types import (
    Enumerator,
    ParameterConstraints,
    Partitioner,
    Perf,
    PerfModel,
    PlanLoader,
    PlannerError,
    PlannerErrorType,
    Proposer,
    ShardingOption,
    Stats,
    Storage,
    StorageReservation,
    Topology,
    hash_planner_context_inputs,
    hash_planner_context_inputs_str,
)
from torchrec_b200.distributed.planner.utils import bytes_to_gb, reset_shard_rank, storage_repr_in_gb
from torchrec_b200.distributed.sharding_plan import get_default_sharders, placement
from torchrec_b200.distributed.types import (
    EmbeddingModuleShardingPlan,
    EnumerableShardingSpec,
    ModuleSharder,
    ParameterSharding,
    ShardingPlan,
    ShardingPlanner,
    ShardingType,
    ShardMetadata,
)

logger: logging.Logger = logging.getLogger(__name__)


def to_sharding_plan(sharding_options: List[ShardingOption], topology: Topology) -> ShardingPlan:
    """Convert placed sharding options into the runtime's ``ShardingPlan``."""
    compute_device = topology.compute_device
    local_size = topology.local_world_size
    plan: Dict[str, EmbeddingModuleShardingPlan] = {}
    for so in sharding_options:
        shards = so.shards
        sharding_type = so.sharding_type
        module_plan = plan.get(so.path, EmbeddingModuleShardingPlan())
        module_plan[so.name] = ParameterSharding(
            sharding_spec=(
                None if sharding_type == ShardingType.DATA_PARALLEL.value
                else EnumerableShardingSpec(
                    [
                        ShardMetadata(shard_sizes=s.size, shard_offsets=s.offset, placement=placement(compute_device, cast(int, s.rank), local_size))
                        for s in shards
                    ]
                )
            ),
            sharding_type=sharding_type,
            compute_kernel=so.compute_kernel,
            ranks=[cast(int, s.rank) for s in shards],
            cache_params=so.cache_params,
            enforce_hbm=so.enforce_hbm,
            stochastic_rounding=so.stochastic_rounding,
            bounds_check_mode=so.bounds_check_mode,
            output_dtype=so.output_dtype,
            key_value_params=so.key_value_params,
        )
        plan[so.path] = module_plan
    return ShardingPlan(plan)


def _merge_plans(best_plans: List[ShardingPlan]) -> ShardingPlan:
    if len(best_plans) == 1:
        return best_plans[0]
    merged = ShardingPlan(plan={})
    for p in best_plans:
        for name, ps in p.plan.items():
            merged.plan.setdefault(name, EmbeddingModuleShardingPlan()).update(ps)  # type: ignore[union-attr]
    return merged


def extract_plan(search_space: List[ShardingOption], loaded_sharding_options: Dict[int, ShardingOption]) -> List[ShardingOption]:
    """Rebuild a stored plan on top of a freshly enumerated search space: every stored option (keyed by ``storage_hash``) lends its
    shards - sizes, offsets, ranks - to the enumerated option with the same key; everything else (tensor, module, input statistics)
    comes from the enumeration, so a stored plan holds no reference to a model.  Raises ``PLAN_LOADING_FAILED`` when two enumerated
    options share a key or the stored plan and the model do not name the same tables.
    Counterpart of ``torchrec/distributed/planner/planners.py:121-197``."""
    by_key: Dict[int, ShardingOption] = {}
    for option in search_space:
        key = option.storage_hash()
        if key in by_key:
            raise PlannerError(f"two sharding options of the search space share the storage hash {key}: {by_key[key].fqn}, {option.fqn}",
                               PlannerErrorType.PLAN_LOADING_FAILED)
        by_key[key] = option
    rebuilt: List[ShardingOption] = []
    for key, stored in loaded_sharding_options.items():
        option = by_key.get(key)
        if option is None:
            continue
        fresh = copy.deepcopy(option)
        fresh.shards = copy.deepcopy(stored.shards)
        rebuilt.append(fresh)
    tables = {o.fqn for o in search_space}
    covered = {o.fqn for o in rebuilt}
    if len(rebuilt) != len(loaded_sharding_options) or covered != tables:
        missing = sorted(tables - covered)
        raise PlannerError(
            f"the stored plan does not fit this model: {len(loaded_sharding_options)} stored options, {len(rebuilt)} matched, "
            f"tables without a stored option: {missing}", PlannerErrorType.PLAN_LOADING_FAILED)
    return rebuilt


class EmbeddingPlannerBase(ShardingPlanner):
    """What every embedding planner here shares: the topology (default: the current world), the batch size, the enumerator, the
    storage reservation, the report sinks, constraints, callbacks and the time limit; ``collective_plan`` (rank 0 plans, everyone
    receives the result) and the fingerprint of the planner's inputs.  Counterpart of ``torchrec/distributed/planner/planners.py:200-340``."""

    def __init__(
        self,
        topology: Optional[Topology] = None,
        batch_size: Optional[int] = None,
        enumerator: Optional[Enumerator] = None,
        storage_reservation: Optional[StorageReservation] = None,
        stats: Optional[Union[Stats, List[Stats]]] = None,
        constraints: Optional[Dict[str, ParameterConstraints]] = None,
        debug: bool = True,
        callbacks: Optional[List[Callable[[List[ShardingOption]], List[ShardingOption]]]] = None,
        timeout_seconds: Optional[int] = None,
        heuristical_storage_reservation_percentage: float = 0.15,
    ) -> None:
        if topology is None:
            world = dist.get_world_size() if dist.is_initialized() else 1
            topology = Topology(local_world_size=get_local_size(world) if dist.is_initialized() else 1, world_size=world,
                                compute_device="cuda" if torch.cuda.is_available() else "cpu")
        self._topology: Topology = topology
        self._batch_size: int = batch_size if batch_size else BATCH_SIZE
        self._constraints = constraints
        self._enumerator: Enumerator = enumerator if enumerator else EmbeddingEnumerator(topology=topology, batch_size=self._batch_size, constraints=constraints)
        self._storage_reservation: StorageReservation = (
            storage_reservation if storage_reservation else HeuristicalStorageReservation(percentage=heuristical_storage_reservation_percentage))
        if stats is not None:
            self._stats: List[Stats] = [stats] if not isinstance(stats, list) else stats
        else:
            from torchrec_b200.distributed.planner.stats import EmbeddingStats

            self._stats = [EmbeddingStats()]
        self._debug = debug
        self._callbacks = [] if callbacks is None else callbacks
        if timeout_seconds is not None:
            assert timeout_seconds > 0, "Timeout must be positive"
        self._timeout_seconds = timeout_seconds

    def collective_plan(self, module: nn.Module, sharders: Optional[List[ModuleSharder[nn.Module]]] = None,
                        pg: Optional[dist.ProcessGroup] = None) -> ShardingPlan:
        """Plan on rank 0 and broadcast."""
        if pg is None:
            assert dist.is_initialized(), "The default process group is not yet initialized. Call torch.distributed.init_process_group first."
            pg = dist.GroupMember.WORLD
        if sharders is None:
            sharders = get_default_sharders()
        return invoke_on_rank_and_broadcast_result(pg, 0, self.plan, module, sharders)

    def hash_planner_context_inputs(self) -> int:
        return hash_planner_context_inputs(self._topology, self._batch_size, self._enumerator, self._storage_reservation, self._constraints)

    def hash_planner_context_inputs_str(self) -> str:
        return hash_planner_context_inputs_str(self._topology, self._batch_size, self._enumerator, self._storage_reservation, self._constraints)


class EmbeddingShardingPlanner(EmbeddingPlannerBase):
    """Searches for the sharding plan with the lowest estimated step time that fits in memory.

    Args:
        topology: devices to plan for (default: the current world, 180 GB HBM each).
        batch_size: per-rank batch size the estimators assume.
        enumerator / storage_reservation / proposer / partitioner / performance_model / stats: plug-ins.
        constraints: per-table restrictions and input statistics.
        debug: print the full plan report.
        plan_loader: source of a plan computed earlier; when it returns one made for the same inputs (fingerprint check), the search
            is skipped and the stored placement is used.
    """

    def __init__(
        self,
        topology: Optional[Topology] = None,
        batch_size: Optional[int] = None,
        enumerator: Optional[Enumerator] = None,
        storage_reservation: Optional[StorageReservation] = None,
        proposer: Optional[Union[Proposer, List[Proposer]]] = None,
        partitioner: Optional[Partitioner] = None,
        performance_model: Optional[PerfModel] = None,
        stats: Optional[Union[Stats, List[Stats]]] = None,
        constraints: Optional[Dict[str, ParameterConstraints]] = None,
        debug: bool = True,
        callbacks: Optional[List[Callable[[List[ShardingOption]], List[ShardingOption]]]] = None,
        timeout_seconds: Optional[int] = None,
        refine_steps: Optional[int] = None,
        plan_loader: Optional[PlanLoader] = None,
    ) -> None:
        super().__init__(topology=topology, batch_size=batch_size, enumerator=enumerator, storage_reservation=storage_reservation, stats=stats,
                         constraints=constraints, debug=debug, callbacks=callbacks, timeout_seconds=timeout_seconds)
        topology = self._topology
        self._partitioner: Partitioner = partitioner if partitioner else GreedyPerfPartitioner()
        if proposer:
            self._proposers: List[Proposer] = [proposer] if not isinstance(proposer, list) else proposer
        else:
            self._proposers = [GridSearchProposer(), GreedyProposer(), GreedyProposer(use_depth=False), UniformProposer()]
        self._perf_model: PerfModel = performance_model if performance_model else NoopPerfModel(topology=topology)
        # local search after the proposers (see _refine): on with the default proposers, off when the caller chose the proposers
        self._refine_steps: int = (16 if not proposer else 0) if refine_steps is None else refine_steps
        self._refine_width: int = 2
        self._refine_seconds: float = 10.0
        self._num_proposals: int = 0
        self._num_plans: int = 0
        self._best_plan: Optional[List[ShardingOption]] = None
        self.plan_loader: Optional[PlanLoader] = plan_loader

    def _load_stored_plan(self, options: List[ShardingOption]) -> Optional[List[ShardingOption]]:
        """The stored placement rebuilt over ``options``; None without a loader or when the loader has nothing.  A plan stored for
        other inputs (topology, batch size, constraints, ...) is refused."""
        if self.plan_loader is None:
            return None
        stored_for = self.plan_loader.plan_context_hash()
        current = self.hash_planner_context_inputs_str()
        if stored_for is not None and stored_for != current:
            plan_id = getattr(self.plan_loader, "get_plan_id", lambda: None)()
            raise PlannerError(
                f"stored plan {plan_id} was computed for other planner inputs (stored {stored_for}, current {current}); it cannot be "
                "shown to be valid for this model and topology", PlannerErrorType.PLANNER_INPUT_CONTEXT_MISMATCH)
        stored = self.plan_loader.load()
        if not stored:
            return None
        return extract_plan(options, stored)

    def plan(self, module: nn.Module, sharders: Optional[List[ModuleSharder[nn.Module]]] = None) -> ShardingPlan:
        """Search: every proposer suggests complete plans; each new suggestion is placed on devices by the partitioner and
        rated by the perf model, and the proposer hears how it went.  The best rated placement wins."""
        sharders = sharders if sharders is not None else get_default_sharders()
        search = _Search(self._timeout_seconds)
        self._num_proposals = self._num_plans = 0
        budget = self._storage_reservation.reserve(topology=self._topology, batch_size=self._batch_size, module=module, sharders=sharders,
                                                   constraints=self._constraints)
        options = self._enumerator.enumerate(module=module, sharders=sharders)
        if not options:
            return ShardingPlan({})
        stored = self._load_stored_plan(options)
        if stored is not None:
            search.note_success(stored, 0.0)
        for proposer in ([] if stored is not None else self._proposers):
            proposer.load(search_space=options, enumerator=self._enumerator)
        for proposer in ([] if stored is not None else self._proposers):
            while not search.out_of_time():
                proposal = proposer.propose()
                if not proposal:
                    break
                self._try_proposal(search, proposer, proposal, budget)
            if search.out_of_time():
                break
        if stored is None and search.best_plan is not None and self._refine_steps > 0:
            self._refine(search, options, budget)
        if search.best_plan is None:
            raise self._no_plan_error(search, budget)
        plan = search.best_plan
        for callback in self._callbacks:
            plan = callback(plan)
        self._best_plan = plan
        result = to_sharding_plan(plan, self._topology)
        elapsed = time.perf_counter() - search.started
        for sink in self._stats:
            sink.log(sharding_plan=result, topology=self._topology, batch_size=self._batch_size, storage_reservation=self._storage_reservation,
                     num_proposals=self._num_proposals, num_plans=self._num_plans, run_time=elapsed, best_plan=plan,
                     constraints=self._constraints, sharders=sharders, enumerator=self._enumerator, debug=self._debug)
        return result

    def _try_proposal(self, search: "_Search", proposer: Optional[Proposer], proposal: List[ShardingOption], budget: Topology) -> Optional[float]:
        """Place and rate one proposal (or replay the verdict if it was seen before); returns the rating, None if it does not fit."""
        key = tuple(sorted(hash(o) for o in proposal))
        known = search.seen.get(key)
        if known is not None:  # another proposer already suggested exactly this: replay the verdict
            ok, placed, rating = known
            if proposer is not None:
                proposer.feedback(partitionable=ok, plan=placed, perf_rating=rating, storage_constraint=budget)
            return rating
        self._num_proposals += 1
        rating: Optional[float] = None
        try:
            placed = self._partitioner.partition(proposal=proposal, storage_constraint=budget)
        except PlannerError as err:
            search.note_failure(err, proposal)
            search.seen[key] = (False, proposal, None)
            if proposer is not None:
                proposer.feedback(partitionable=False, plan=proposal, storage_constraint=budget)
        else:
            self._num_plans += 1
            rating = self._perf_model.rate(plan=placed)
            search.note_success(placed, rating)
            search.seen[key] = (True, placed, rating)
            if proposer is not None:
                proposer.feedback(partitionable=True, plan=placed, perf_rating=rating, storage_constraint=budget)
        search.last_proposal = copy.deepcopy(proposal)
        reset_shard_rank(proposal)  # the option objects are shared between proposals: forget this placement
        return rating

    def _refine(self, search: "_Search", options: List[ShardingOption], budget: Topology) -> None:
        """Local search around the proposers' best plan: while the rating improves, take the most loaded rank, and for its most
        expensive tables try every other way of sharding that one table (all other tables keep their option; the partitioner
        places the whole proposal again).  The proposers walk the search space along one ordering of the options, so a plan
        that differs from their best one in a single table (one heavy table-wise table split row-wise, say) is often never
        suggested; this step finds it.  The reference's planner stops after the proposers
        (torchrec/distributed/planner/planners.py:520-640)."""
        def shape(o: ShardingOption):
            return (o.fqn, o.sharding_type, o.compute_kernel, tuple((tuple(s.size), tuple(s.offset)) for s in o.shards), o.cache_params)

        unplaced = {shape(o): o for o in options}
        by_table: Dict[str, List[ShardingOption]] = {}
        for o in options:
            by_table.setdefault(o.fqn, []).append(o)
        deadline = time.perf_counter() + self._refine_seconds
        for _ in range(self._refine_steps):
            base = [unplaced.get(shape(o)) for o in cast(List[ShardingOption], search.best_plan)]
            if any(o is None for o in base):  # a callback or proposer changed the options: nothing to vary safely
                return
            load: Dict[int, float] = {}
            for o in cast(List[ShardingOption], search.best_plan):
                for s in o.shards:
                    load[cast(int, s.rank)] = load.get(cast(int, s.rank), 0.0) + cast(Perf, s.perf).total
            worst = max(load, key=lambda r: load[r])
            on_worst = sorted(((max(cast(Perf, s.perf).total for s in o.shards if s.rank == worst), i)
                               for i, o in enumerate(cast(List[ShardingOption], search.best_plan)) if any(s.rank == worst for s in o.shards)), reverse=True)
            before = search.best_rating
            for _, i in on_worst[: self._refine_width]:
                for alt in by_table[cast(ShardingOption, base[i]).fqn]:
                    if alt is base[i]:
                        continue
                    if search.out_of_time() or time.perf_counter() > deadline:
                        return
                    self._try_proposal(search, None, [alt if j == i else cast(ShardingOption, o) for j, o in enumerate(base)], budget)
            if search.best_rating >= before:
                return

    def _no_plan_error(self, search: "_Search", budget: Topology) -> PlannerError:
        def total(devices) -> Storage:
            acc = Storage(0, 0)
            for d in devices:
                acc = acc + d.storage
            return acc

        hardware, available, needed = total(self._topology.devices), total(budget.devices), search.smallest_failure
        reservation = self._storage_reservation
        advice = [
            f"Planner evaluated {self._num_proposals} proposals.",
            "Possible solutions:",
            f"  1) Increase the number of devices ({self._topology.world_size})",
            "  2) Reduce the model size (",
            f"\t  Global storage: {round(bytes_to_gb(hardware.hbm), 3)} GB, ",
            f"\t  Per rank hardware memory: {storage_repr_in_gb(self._topology.devices[0].storage)}, ",
            f"\t  Available for model parallel: {round(bytes_to_gb(available.hbm), 3)} GB, ",
            f"\t  Requirement for model parallel: {round(bytes_to_gb(needed.hbm), 3)} GB)",
            f"  3) Reduce local batch size ({self._batch_size})",
            "  4) Remove planner constraints that might be reducing search space or available storage",
        ]
        tail = f"Last planner error: \n\t{search.last_error}\n"
        if not needed.fits_in(available):
            if isinstance(reservation, HeuristicalStorageReservation):
                advice += [
                    f"\t  Storage reservation percentage: {reservation._percentage}, ",
                    f"\t  Per rank reservation for dense storage: {storage_repr_in_gb(reservation._dense_storage)}, ",
                    f"\t  Per rank reservation for kjt storage: {storage_repr_in_gb(reservation._kjt_storage)}, ",
                ]
            return PlannerError(error_type=PlannerErrorType.INSUFFICIENT_STORAGE,
                                message="Unable to find a plan for this model because of insufficient storage. \n" + "\n".join(advice) + "\n" + tail)
        return PlannerError(error_type=PlannerErrorType.STRICT_CONSTRAINTS,
                            message="Unable to find a plan for this model because of the strict constraints. \n" + "\n".join(advice) + "\n" + tail)


class _Search:
    """Book-keeping of one ``plan`` call: verdicts by proposal, the best placement so far, what failed and why."""

    def __init__(self, timeout_seconds: Optional[int]) -> None:
        self.started = time.perf_counter()
        self.timeout = timeout_seconds
        self.seen: Dict[Tuple[int, ...], Tuple[bool, Optional[List[ShardingOption]], Optional[float]]] = {}
        self.best_plan: Optional[List[ShardingOption]] = None
        self.best_rating: float = MAX_SIZE
        self.smallest_failure = Storage(MAX_SIZE, MAX_SIZE)
        self.last_error: Optional[PlannerError] = None
        self.last_proposal: List[ShardingOption] = []

    def out_of_time(self) -> bool:
        return self.timeout is not None and time.perf_counter() - self.started > self.timeout

    def note_success(self, placed: List[ShardingOption], rating: float) -> None:
        if rating < self.best_rating:
            self.best_rating, self.best_plan = rating, copy.deepcopy(placed)

    def note_failure(self, err: PlannerError, proposal: List[ShardingOption]) -> None:
        self.last_error = err
        need = Storage(0, 0)
        for option in proposal:
            for shard in option.shards:
                need = need + cast(Storage, shard.storage)
        if need < self.smallest_failure:
            self.smallest_failure = need


class HeteroEmbeddingShardingPlanner(ShardingPlanner):
    """Plans over several device groups (e.g. ``cuda`` and ``cpu``) with one planner per group; a table's
    ``ParameterConstraints.device_group`` selects the group it may be placed on."""

    def __init__(self, topology_groups: Optional[Dict[str, Topology]] = None, batch_size: Optional[int] = None,
                 enumerators: Optional[Dict[str, Enumerator]] = None, storage_reservations: Optional[Dict[str, StorageReservation]] = None,
                 proposers: Optional[Dict[str, Union[Proposer, List[Proposer]]]] = None, partitioners: Optional[Dict[str, Partitioner]] = None,
                 performance_models: Optional[Dict[str, PerfModel]] = None, stats: Optional[Dict[str, Union[Stats, List[Stats]]]] = None,
                 constraints: Optional[Dict[str, ParameterConstraints]] = None, debug: bool = True,
                 callbacks: Optional[List[Callable[[List[ShardingOption]], List[ShardingOption]]]] = None) -> None:
        default_device = "cuda" if torch.cuda.is_available() else "cpu"
        if topology_groups is None:
            world = dist.get_world_size() if dist.is_initialized() else 1
            topology_groups = {default_device: Topology(local_world_size=get_local_size(world) if dist.is_initialized() else 1, world_size=world, compute_device=default_device)}
        self._topology_groups = topology_groups
        self._planners: Dict[str, EmbeddingShardingPlanner] = {}
        for group, topology in topology_groups.items():
            self._planners[group] = EmbeddingShardingPlanner(
                topology=topology, batch_size=batch_size, enumerator=enumerators.get(group) if enumerators else None,
                storage_reservation=storage_reservations.get(group) if storage_reservations else None,
                proposer=proposers.get(group) if proposers else None, partitioner=partitioners.get(group) if partitioners else None,
                performance_model=performance_models.get(group) if performance_models else None, stats=stats.get(group) if stats else None,
                constraints=constraints, debug=debug, callbacks=callbacks,
            )

    def collective_plan(self, module: nn.Module, sharders: Optional[List[ModuleSharder[nn.Module]]] = None,
                        pg: Optional[dist.ProcessGroup] = None) -> ShardingPlan:
        if pg is None:
            pg = dist.GroupMember.WORLD
        if sharders is None:
            sharders = get_default_sharders()
        return invoke_on_rank_and_broadcast_result(pg, 0, self.plan, module, sharders)

    def plan(self, module: nn.Module, sharders: Optional[List[ModuleSharder[nn.Module]]] = None) -> ShardingPlan:
        if sharders is None:
            sharders = get_default_sharders()
        return _merge_plans([p.plan(module, sharders) for p in self._planners.values()])
