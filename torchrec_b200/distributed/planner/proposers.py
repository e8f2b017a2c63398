"""Proposers: walk the search space and emit candidate plans (one option per table).
Counterpart of ``torchrec/distributed/planner/proposers.py``.
"""
from __future__ import annotations

import copy
import itertools
import logging
from decimal import Decimal
from typing import Dict, List, Optional, Set, Tuple, Union, cast

import torch

from torchrec_b200.distributed.embedding_types import EmbeddingComputeKernel
from torchrec_b200.distributed.planner.types import Enumerator, Perf, Proposer, ShardingOption, Topology
from torchrec_b200.distributed.planner.utils import BinarySearchPredicate, bytes_to_gb, prod

logger: logging.Logger = logging.getLogger(__name__)

MAX_PROPOSALS: int = int(1e4)


def _sharding_option_score(so: ShardingOption, use_depth: bool = True) -> float:
    return max(cast(Perf, s.perf).total for s in so.shards) if use_depth else sum(cast(Perf, s.perf).total for s in so.shards)


class GreedyProposer(Proposer):
    """Start from the cheapest option of every table; after an infeasible plan, replace the option that uses
    the most HBM by the next cheapest of its table.  ``use_depth``: rank options by their slowest shard
    (else by the sum over shards)."""

    def __init__(self, use_depth: bool = True, threshold: Optional[int] = None) -> None:
        self._use_depth = use_depth
        self._threshold = threshold if threshold else None
        self._sharding_options_by_fqn: Dict[str, List[ShardingOption]] = {}
        self._current_proposal: Dict[str, int] = {}
        self._best_perf_rating: float = float("inf")
        self._num_inferior_perf: int = 0

    def load(self, search_space: List[ShardingOption], enumerator: Optional[Enumerator] = None) -> None:
        self._reset()
        for so in search_space:
            self._sharding_options_by_fqn.setdefault(so.fqn, []).append(so)
        for options in self._sharding_options_by_fqn.values():
            options.sort(key=lambda x: _sharding_option_score(x, self._use_depth))
        self._current_proposal = {fqn: 0 for fqn in self._sharding_options_by_fqn.keys()}

    def _reset(self) -> None:
        self._sharding_options_by_fqn = {}
        self._current_proposal = {}

    def propose(self) -> Optional[List[ShardingOption]]:
        if self._current_proposal:
            return [self._sharding_options_by_fqn[fqn][i] for fqn, i in self._current_proposal.items()]
        return None

    def _patience_ran_out(self, perf_rating: Optional[float]) -> bool:
        """With a threshold: stop after that many proposals in a row that did not improve on the best rating seen."""
        if not (self._threshold and perf_rating):
            return False
        improved = perf_rating < self._best_perf_rating
        self._best_perf_rating = min(self._best_perf_rating, perf_rating)
        self._num_inferior_perf = 0 if improved else self._num_inferior_perf + 1
        return self._num_inferior_perf > self._threshold

    def feedback(self, partitionable: bool, plan: Optional[List[ShardingOption]] = None, perf_rating: Optional[float] = None,
                 storage_constraint: Optional[Topology] = None) -> None:
        if self._patience_ran_out(perf_rating):
            self._current_proposal = {}
            return
        # the table whose current option needs the most HBM moves on to its next cheapest option; when it has none left, the search ends
        chosen = self._current_proposal

        def hbm_of(fqn: str) -> int:
            return self._sharding_options_by_fqn[fqn][chosen[fqn]].total_storage.hbm

        heaviest = max(chosen, key=hbm_of)
        if chosen[heaviest] + 1 < len(self._sharding_options_by_fqn[heaviest]):
            chosen[heaviest] += 1
        else:
            self._current_proposal = {}


class UniformProposer(Proposer):
    """Plans in which every table uses the same sharding type."""

    def __init__(self, use_depth: bool = True) -> None:
        self._use_depth = use_depth
        self._grouped_sharding_options: List[List[ShardingOption]] = []
        self._proposal_index = 0

    def load(self, search_space: List[ShardingOption], enumerator: Optional[Enumerator] = None) -> None:
        self._reset()
        all_fqns = {so.fqn for so in search_space}
        by_type_fqn: Dict[str, Dict[str, List[ShardingOption]]] = {}
        for so in search_space:
            by_type_fqn.setdefault(so.sharding_type, {}).setdefault(so.fqn, []).append(so)
        for sharding_type, by_fqn in by_type_fqn.items():
            if by_fqn.keys() == all_fqns:
                self._grouped_sharding_options.append([sorted(opts, key=lambda x: _sharding_option_score(x, self._use_depth))[0] for opts in by_fqn.values()])

    def _reset(self) -> None:
        self._grouped_sharding_options = []
        self._proposal_index = 0

    def propose(self) -> Optional[List[ShardingOption]]:
        if self._proposal_index < len(self._grouped_sharding_options):
            return self._grouped_sharding_options[self._proposal_index]
        return None

    def feedback(self, partitionable: bool, plan=None, perf_rating=None, storage_constraint=None) -> None:
        self._proposal_index += 1


class GridSearchProposer(Proposer):
    """Exhaustive product of the options of all tables, when that product is small enough."""

    def __init__(self, max_proposals: int = MAX_PROPOSALS) -> None:
        self._max_proposals = max_proposals
        self._sharding_options_by_fqn: Dict[str, List[ShardingOption]] = {}
        self._proposal_index = 0
        self._proposals: List[List[int]] = []

    def load(self, search_space: List[ShardingOption], enumerator: Optional[Enumerator] = None) -> None:
        self._reset()
        for so in search_space:
            self._sharding_options_by_fqn.setdefault(so.fqn, []).append(so)
        for options in self._sharding_options_by_fqn.values():
            options.sort(key=lambda x: _sharding_option_score(x))
        total = prod(len(x) for x in self._sharding_options_by_fqn.values())
        if total > self._max_proposals:
            logger.info(f"Skipping grid search proposer as there are too many proposals ({total} > {self._max_proposals})")
            return
        self._proposals = [list(p) for p in itertools.product(*[range(len(x)) for x in self._sharding_options_by_fqn.values()])]

    def _reset(self) -> None:
        self._sharding_options_by_fqn = {}
        self._proposal_index = 0
        self._proposals = []

    def propose(self) -> Optional[List[ShardingOption]]:
        if self._proposals and self._proposal_index < len(self._proposals):
            idx = self._proposals[self._proposal_index]
            return [opts[i] for opts, i in zip(self._sharding_options_by_fqn.values(), idx)]
        return None

    def feedback(self, partitionable: bool, plan=None, perf_rating=None, storage_constraint=None) -> None:
        self._proposal_index += 1


class DynamicProgrammingProposer(Proposer):
    """Knapsack over discretised HBM: for every memory budget, the set of options (one per table) with the
    lowest summed perf.  Proposals are emitted from the tightest feasible budget upwards."""

    def __init__(self, hbm_bins_per_device: int = 100) -> None:
        self._inited = False
        self._hbm_bins_per_device = max(hbm_bins_per_device, 1)
        self._sharding_options_by_fqn: Dict[str, List[ShardingOption]] = {}
        self._proposal_list: List[List[int]] = []
        self._current_proposal = -1

    def load(self, search_space: List[ShardingOption], enumerator: Optional[Enumerator] = None) -> None:
        self._reset()
        for so in sorted(search_space, key=lambda x: x.total_storage.hbm):
            self._sharding_options_by_fqn.setdefault(so.fqn, []).append(so)

    def _reset(self) -> None:
        self._sharding_options_by_fqn = {}
        self._proposal_list = []
        self._current_proposal = -1

    def propose(self) -> Optional[List[ShardingOption]]:
        if not self._inited:
            return [opts[0] for opts in self._sharding_options_by_fqn.values()]
        if self._current_proposal >= 0:
            idx = self._proposal_list[self._current_proposal]
            return [self._sharding_options_by_fqn[fqn][i] for fqn, i in zip(self._sharding_options_by_fqn.keys(), idx)]
        return None

    def feedback(self, partitionable: bool, plan=None, perf_rating=None, storage_constraint: Optional[Topology] = None) -> None:
        if not self._inited:
            self._inited = True
            assert storage_constraint is not None
            hbm_total = sum(d.storage.hbm for d in storage_constraint.devices)
            bin_count = self._hbm_bins_per_device * len(storage_constraint.devices)
            bin_size = max(float(hbm_total) / bin_count, 1.0)
            tables = list(self._sharding_options_by_fqn.values())
            INF = float("inf")
            dp = [[INF] * bin_count for _ in range(len(tables))]
            back = [[(-1, -1)] * bin_count for _ in range(len(tables))]
            for t, opts in enumerate(tables):
                for oi, so in enumerate(opts):
                    need = int(so.total_storage.hbm / bin_size + 0.999)
                    perf = so.total_perf
                    if t == 0:
                        if need < bin_count and dp[0][need] > perf:
                            dp[0][need] = perf
                            back[0][need] = (oi, -1)
                    else:
                        for prev in range(bin_count):
                            if dp[t - 1][prev] == INF:
                                continue
                            cur = prev + need
                            if cur < bin_count and dp[t][cur] > dp[t - 1][prev] + perf:
                                dp[t][cur] = dp[t - 1][prev] + perf
                                back[t][cur] = (oi, prev)
            self._proposal_list = []
            best = INF
            for c in range(bin_count - 1, -1, -1):
                cur_perf = dp[-1][c]
                if cur_perf < best:
                    best = cur_perf
                    idx = [-1] * len(tables)
                    b = c
                    for t in range(len(tables) - 1, -1, -1):
                        idx[t], b = back[t][b]
                    self._proposal_list.append(idx)
            self._current_proposal = len(self._proposal_list) - 1 if self._proposal_list else -1
        else:
            self._current_proposal -= 1


class EmbeddingOffloadScaleupProposer(Proposer):
    """For plans that offload tables (``FUSED_UVM_CACHING``): spend leftover HBM on larger caches.
    After the starting proposal it binary-searches the total cache budget that still partitions."""

    def __init__(self, use_depth: bool = True) -> None:
        self.use_depth = use_depth
        self.enumerator: Optional[Enumerator] = None
        self.starting_proposal: List[ShardingOption] = []
        self.proposal: Optional[List[ShardingOption]] = None
        self.search: Optional[BinarySearchPredicate] = None
        self.best_perf_rating = 1e99

    def load(self, search_space: List[ShardingOption], enumerator: Optional[Enumerator] = None) -> None:
        self.enumerator = enumerator
        by_fqn: Dict[str, List[ShardingOption]] = {}
        for so in search_space:
            by_fqn.setdefault(so.fqn, []).append(so)
        for opts in by_fqn.values():
            opts.sort(key=lambda x: _sharding_option_score(x, self.use_depth))
        self.starting_proposal = [opts[0] for opts in by_fqn.values()]
        self.proposal = copy.deepcopy(self.starting_proposal)

    def propose(self) -> Optional[List[ShardingOption]]:
        return self.proposal

    @staticmethod
    def get_scalable_sharding_options(proposal: List[ShardingOption]) -> List[ShardingOption]:
        return [so for so in proposal if so.compute_kernel == EmbeddingComputeKernel.FUSED_UVM_CACHING.value and so.cache_params is not None]

    def feedback(self, partitionable: bool, plan=None, perf_rating=None, storage_constraint: Optional[Topology] = None) -> None:
        if not self.enumerator or plan is None or not self.get_scalable_sharding_options(plan):
            self.proposal = None
            return
        hbm_available = sum(d.storage.hbm for d in storage_constraint.devices) if storage_constraint else 0
        used = sum(so.total_storage.hbm for so in plan)
        if self.search is None:
            if not partitionable or hbm_available <= used:
                self.proposal = None
                return
            self.search = BinarySearchPredicate(0, hbm_available - used, max((hbm_available - used) // 100, 1))
        budget = self.search.next(partitionable)
        if budget is None:
            self.proposal = None
            return
        self.proposal = self.next_plan(self.starting_proposal, budget, self.enumerator)

    @staticmethod
    def next_plan(starting_proposal: List[ShardingOption], budget: int, enumerator: Optional[Enumerator]) -> Optional[List[ShardingOption]]:
        proposal = copy.deepcopy(starting_proposal)
        scalable = EmbeddingOffloadScaleupProposer.get_scalable_sharding_options(proposal)
        if not scalable:
            return None
        sizes = [prod(so.tensor.shape) * so.tensor.element_size() for so in scalable]
        total = float(sum(sizes))
        for so, sz in zip(scalable, sizes):
            extra = budget * (sz / total)
            clf = min(1.0, (so.cache_params.load_factor or 0.0) + extra / max(sz, 1))
            so.cache_params = copy.copy(so.cache_params)
            so.cache_params.load_factor = clf
            if clf >= 0.9999:
                so.compute_kernel = EmbeddingComputeKernel.FUSED.value
                so.cache_params.load_factor = None
        if enumerator is not None:
            enumerator.populate_estimates(scalable)
        return proposal


def proposers_to_proposals_list(proposers_list: List[Proposer], search_space: List[ShardingOption]) -> List[List[ShardingOption]]:
    """All proposals of all proposers (feedback is always "not partitionable" so each one runs to exhaustion)."""
    def drain(proposer: Proposer):
        proposer.load(search_space=search_space)
        while True:
            proposal = proposer.propose()
            if not proposal:
                return
            yield proposal
            proposer.feedback(partitionable=True)

    distinct: Dict[Tuple[int, ...], List[ShardingOption]] = {}  # keyed by the set of options, first occurrence kept, order of discovery
    for proposer in proposers_list:
        for proposal in drain(proposer):
            distinct.setdefault(tuple(sorted(map(id, proposal))), proposal)
    return list(distinct.values())
