"""Planner: search space, constraints, memory feasibility, balance, determinism (cf. ``torchrec/distributed/planner/tests``)."""
import pytest
import torch
from torch import nn

from torchrec_b200.distributed.embedding_types import EmbeddingComputeKernel
from torchrec_b200.distributed.embeddingbag import EmbeddingBagCollectionSharder
from torchrec_b200.distributed.planner import EmbeddingShardingPlanner, ParameterConstraints, Topology
from torchrec_b200.distributed.planner.enumerators import EmbeddingEnumerator
from torchrec_b200.distributed.planner.partitioners import GreedyPerfPartitioner, MemoryBalancedPartitioner
from torchrec_b200.distributed.planner.proposers import DynamicProgrammingProposer, GreedyProposer, GridSearchProposer, UniformProposer, proposers_to_proposals_list
from torchrec_b200.distributed.planner.storage_reservations import FixedPercentageStorageReservation, HeuristicalStorageReservation
from torchrec_b200.distributed.planner.types import PlannerError, PlannerErrorType
from torchrec_b200.distributed.types import ShardingType
from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection

GB = 1024 ** 3


class _Model(nn.Module):
    def __init__(self, tables):
        super().__init__()
        self.sparse = EmbeddingBagCollection(tables=tables, device=torch.device("meta"))
        self.dense = nn.Linear(8, 8)


def _tables(n=4, rows=1000, dim=64):
    return [EmbeddingBagConfig(name=f"t{i}", embedding_dim=dim, num_embeddings=rows * (i + 1), feature_names=[f"f{i}"]) for i in range(n)]


def _topo(world=2, hbm=8 * GB, local=None):
    return Topology(world_size=world, compute_device="cuda", hbm_cap=hbm, local_world_size=local)


def test_enumerator_covers_sharding_types_and_respects_constraints():
    model = _Model(_tables(2))
    topo = _topo(4, local=2)
    opts = EmbeddingEnumerator(topology=topo, batch_size=128).enumerate(model, [EmbeddingBagCollectionSharder()])
    kinds = {(o.name, o.sharding_type) for o in opts}
    for st in (ShardingType.TABLE_WISE, ShardingType.ROW_WISE, ShardingType.COLUMN_WISE, ShardingType.DATA_PARALLEL, ShardingType.TABLE_ROW_WISE):
        assert ("t0", st.value) in kinds, st
    for o in opts:
        assert o.total_storage.hbm > 0 and o.total_perf > 0, (o.name, o.sharding_type)
        rows = sum(s.size[0] for s in o.shards) if o.sharding_type in (ShardingType.ROW_WISE.value, ShardingType.TABLE_ROW_WISE.value) else None
        if rows is not None:
            assert rows == o.tensor.shape[0]
        if o.sharding_type == ShardingType.COLUMN_WISE.value:
            assert sum(s.size[1] for s in o.shards) == o.tensor.shape[1]
    cons = {"t0": ParameterConstraints(sharding_types=[ShardingType.ROW_WISE.value], compute_kernels=[EmbeddingComputeKernel.FUSED.value]),
            "t1": ParameterConstraints(sharding_types=[ShardingType.COLUMN_WISE.value], min_partition=32)}
    opts = EmbeddingEnumerator(topology=topo, batch_size=128, constraints=cons).enumerate(model, [EmbeddingBagCollectionSharder()])
    assert {o.sharding_type for o in opts if o.name == "t0"} == {ShardingType.ROW_WISE.value}
    assert {o.compute_kernel for o in opts if o.name == "t0"} == {EmbeddingComputeKernel.FUSED.value}
    t1 = [o for o in opts if o.name == "t1"]
    assert t1 and all(o.sharding_type == ShardingType.COLUMN_WISE.value and all(s.size[1] >= 32 for s in o.shards) for o in t1)


def test_plan_places_every_shard_within_memory_and_is_deterministic():
    model = _Model(_tables(6, rows=200_000, dim=128))
    topo = _topo(4)
    plans = []
    for _ in range(2):
        planner = EmbeddingShardingPlanner(topology=_topo(4), batch_size=512, debug=False)
        plans.append(planner.plan(model, [EmbeddingBagCollectionSharder()]))
    a, b = (p.plan["sparse"] for p in plans)
    assert set(a.keys()) == {f"t{i}" for i in range(6)}
    for name in a:
        assert a[name].sharding_type == b[name].sharding_type and a[name].ranks == b[name].ranks
        spec = a[name].sharding_spec
        if spec is not None:
            rows, dim = 200_000 * (int(name[1:]) + 1), 128
            assert sum(s.shard_sizes[0] * s.shard_sizes[1] for s in spec.shards) == rows * dim
    used = [0] * 4
    for name, ps in a.items():
        if ps.sharding_spec is None:
            continue
        for s in ps.sharding_spec.shards:
            r = int(str(s.placement).split("/")[0].split(":")[1])
            used[r] += s.shard_sizes[0] * s.shard_sizes[1] * 4
    assert max(used) < 8 * GB and min(used) > 0


def test_plan_fails_with_a_storage_error_when_nothing_fits():
    model = _Model(_tables(3, rows=4_000_000, dim=128))  # ~2 GB, 4 GB, 6 GB tables (+ optimizer/IO) on 2 x 1 GB
    hbm_only = {f"t{i}": ParameterConstraints(compute_kernels=[EmbeddingComputeKernel.FUSED.value]) for i in range(3)}  # no spill-over to host memory
    planner = EmbeddingShardingPlanner(topology=_topo(2, hbm=1 * GB), batch_size=512, debug=False, constraints=hbm_only)
    with pytest.raises(PlannerError) as e:
        planner.plan(model, [EmbeddingBagCollectionSharder()])
    assert e.value.error_type in (PlannerErrorType.INSUFFICIENT_STORAGE, PlannerErrorType.PARTITION)


def test_big_table_is_split_when_it_does_not_fit_on_one_device():
    tables = [EmbeddingBagConfig(name="big", embedding_dim=128, num_embeddings=6_000_000, feature_names=["f"])]  # 3 GB of weights
    planner = EmbeddingShardingPlanner(topology=_topo(4, hbm=2 * GB), batch_size=512, debug=False, storage_reservation=FixedPercentageStorageReservation(0.1),
                                       constraints={"big": ParameterConstraints(compute_kernels=[EmbeddingComputeKernel.FUSED.value])})
    ps = planner.plan(_Model(tables), [EmbeddingBagCollectionSharder()]).plan["sparse"]["big"]
    assert ps.sharding_type in (ShardingType.ROW_WISE.value, ShardingType.COLUMN_WISE.value, ShardingType.TABLE_ROW_WISE.value, ShardingType.GRID_SHARD.value)
    assert len(ps.ranks) >= 2


def test_proposers_and_partitioners():
    model = _Model(_tables(3))
    topo = _topo(2)
    space = EmbeddingEnumerator(topology=topo, batch_size=128).enumerate(model, [EmbeddingBagCollectionSharder()])
    for proposer in (GreedyProposer(), UniformProposer(), GridSearchProposer(), DynamicProgrammingProposer()):
        proposer.load(space)
        first = proposer.propose()
        assert first is not None and sorted(o.name for o in first) == ["t0", "t1", "t2"], type(proposer).__name__
        proposer.feedback(partitionable=True, plan=first, perf_rating=1.0, storage_constraint=topo)
    uni = UniformProposer()
    uni.load(space)
    seen = set()
    while (p := uni.propose()) is not None:
        kinds = {o.sharding_type for o in p}
        assert len(kinds) == 1
        seen |= kinds
        uni.feedback(True)
    assert ShardingType.TABLE_WISE.value in seen and ShardingType.ROW_WISE.value in seen
    assert len(proposers_to_proposals_list([GreedyProposer(), UniformProposer()], space)) >= 2
    greedy = GreedyProposer()
    greedy.load(space)
    proposal = greedy.propose()
    for part in (GreedyPerfPartitioner(), MemoryBalancedPartitioner()):
        placed = part.partition([o for o in __import__("copy").deepcopy(proposal)], _topo(2))
        for o in placed:
            assert all(s.rank is not None and 0 <= s.rank < 2 for s in o.shards)
    with pytest.raises(PlannerError):
        GreedyPerfPartitioner().partition(__import__("copy").deepcopy(proposal), _topo(2, hbm=1024))


def test_storage_reservations_shrink_the_topology():
    model = _Model(_tables(2))
    topo = _topo(2, hbm=10 * GB)
    fixed = FixedPercentageStorageReservation(0.2).reserve(topo, 512, model, [EmbeddingBagCollectionSharder()])
    assert fixed.devices[0].storage.hbm == int(10 * GB * 0.8)
    heur = HeuristicalStorageReservation(percentage=0.15).reserve(_topo(2, hbm=10 * GB), 512, model, [EmbeddingBagCollectionSharder()])
    assert heur.devices[0].storage.hbm < int(10 * GB * 0.85)
    assert topo.devices[0].storage.hbm == 10 * GB  # the input topology is untouched


def test_plan_report_lists_every_table():
    from torchrec_b200.distributed.planner.stats import EmbeddingStats

    stats = EmbeddingStats()
    planner = EmbeddingShardingPlanner(topology=_topo(2), batch_size=256, debug=True, stats=stats)
    planner.plan(_Model(_tables(3)), [EmbeddingBagCollectionSharder()])
    report = stats.report()
    for t in ("t0", "t1", "t2"):
        assert t in report
    assert "Rank" in report or "rank" in report


def test_perf_estimator_matches_hand_computed_numbers():
    """The wall-time model on round numbers, worked out by hand here (cf. ``torchrec/distributed/planner/tests/test_shard_estimators.py``):
    bandwidths of 1000 bytes/ms for memory and 100 bytes/ms for the links make every term readable."""
    from torchrec_b200.distributed.planner.shard_estimators import EmbeddingPerfEstimator
    from torchrec_b200.distributed.planner.types import BasicCommsBandwidths

    common = dict(
        compute_kernel="fused", compute_device="cuda", batch_sizes=[10], world_size=2, local_world_size=2, input_lengths=[4.0],
        input_data_type_size=8.0, table_data_type_size=4.0, output_data_type_size=4.0, fwd_a2a_comm_data_type_size=4.0,
        bwd_a2a_comm_data_type_size=4.0, fwd_sr_comm_data_type_size=4.0, bwd_sr_comm_data_type_size=4.0, num_poolings=[1.0],
        hbm_mem_bw=1250.0, ddr_mem_bw=100.0, hbm_to_ddr_mem_bw=10.0, comms_bandwidths=BasicCommsBandwidths(inter_host_bw=10.0, intra_host_bw=100.0),
        bwd_compute_multiplier=2.0, weighted_feature_bwd_compute_multiplier=1.0, is_pooled=True,
    )
    # fused kernels read at 0.8 x HBM = 1000 bytes/ms; dim 128 carries no narrow-row penalty
    (tw,) = EmbeddingPerfEstimator.perf_func_emb_wall_time(shard_sizes=[[1000, 128]], sharding_type="table_wise", **common)
    ids = 4 * 10 * 2                      # pooling x batch x world: the owner looks up the global batch
    id_bytes, row_bytes, out_bytes = ids * 8, ids * 128 * 4, 10 * 2 * 128 * 4
    assert tw.fwd_compute == pytest.approx((id_bytes + row_bytes + out_bytes) / 1000.0)
    assert tw.fwd_comms == pytest.approx(out_bytes * 0.5 / 100.0)     # half of the pooled rows leave the owner
    assert tw.bwd_compute == pytest.approx(2.0 * tw.fwd_compute)
    assert tw.bwd_comms == pytest.approx(tw.fwd_comms)
    # exchanges fused into the lookup kernels overlap with them: the slower of the two sides is the cost
    from torchrec_b200.distributed.planner.constants import FUSED_DIST_OVERLAP

    overlapped = max(tw.fwd_compute, tw.fwd_comms) + max(tw.bwd_compute, tw.bwd_comms)
    assert tw.total == pytest.approx(overlapped if FUSED_DIST_OVERLAP else tw.fwd_compute + tw.fwd_comms + tw.bwd_compute + tw.bwd_comms)
    # row-wise over 2 shards: half the ids per shard, a partial row for every bag of the global batch from every shard
    (rw, rw2) = EmbeddingPerfEstimator.perf_func_emb_wall_time(shard_sizes=[[500, 128], [500, 128]], sharding_type="row_wise", **common)
    assert rw.fwd_compute == pytest.approx((id_bytes / 2 + row_bytes / 2 + out_bytes) / 1000.0)
    assert rw.fwd_comms == pytest.approx(out_bytes * 0.5 / 100.0)
    assert rw2.total == pytest.approx(rw.total)
    # data parallel: local batch only, no exchange forward, the whole table's gradient all-reduced backward
    (dp,) = EmbeddingPerfEstimator.perf_func_emb_wall_time(shard_sizes=[[1000, 128]], sharding_type="data_parallel", **common)
    local_ids = 4 * 10
    assert dp.fwd_comms == 0
    assert dp.fwd_compute == pytest.approx((local_ids * 8 + local_ids * 128 * 4 + 10 * 128 * 4) / 1000.0)
    assert dp.bwd_comms == pytest.approx(1000 * 128 * 4 / 100.0)
    # narrow rows waste part of every memory transaction
    (narrow,) = EmbeddingPerfEstimator.perf_func_emb_wall_time(shard_sizes=[[1000, 16]], sharding_type="table_wise", **common)
    assert narrow.fwd_compute > (id_bytes + ids * 32 * 4 + 10 * 2 * 16 * 4) / 1000.0
    # inference has no backward
    (inf,) = EmbeddingPerfEstimator.perf_func_emb_wall_time(shard_sizes=[[1000, 128]], sharding_type="table_wise", is_inference=True, **common)
    assert inf.bwd_compute == 0 and inf.bwd_comms == 0 and inf.fwd_compute == pytest.approx(tw.fwd_compute)


def test_perf_estimator_tracks_the_measured_lookup():
    """Calibration against a measured kernel time on B200: the pooled forward over 14.0 M ids x 512 B rows took 1.31 ms; the model's
    forward-compute figure for the same work on the default topology must land within a factor 1.5 of it."""
    from torchrec_b200.distributed.planner.constants import HBM_MEM_BW
    from torchrec_b200.distributed.planner.shard_estimators import EmbeddingPerfEstimator
    from torchrec_b200.distributed.planner.types import BasicCommsBandwidths

    (p,) = EmbeddingPerfEstimator.perf_func_emb_wall_time(
        shard_sizes=[[40_000_000, 128]], compute_kernel="fused", compute_device="cuda", sharding_type="table_wise", batch_sizes=[65536], world_size=1,
        local_world_size=1, input_lengths=[214.0], input_data_type_size=4.0, table_data_type_size=4.0, output_data_type_size=2.0,
        fwd_a2a_comm_data_type_size=2.0, bwd_a2a_comm_data_type_size=2.0, fwd_sr_comm_data_type_size=2.0, bwd_sr_comm_data_type_size=2.0,
        num_poolings=[1.0], hbm_mem_bw=HBM_MEM_BW, ddr_mem_bw=1.0, hbm_to_ddr_mem_bw=1.0, comms_bandwidths=BasicCommsBandwidths(),
        bwd_compute_multiplier=2.0, weighted_feature_bwd_compute_multiplier=1.0, is_pooled=True)
    assert 1.31 / 1.5 < p.fwd_compute < 1.31 * 1.5, p.fwd_compute


def test_local_refinement_never_rates_worse_and_balances_a_skewed_model():
    """One table with a far larger pooling factor than the rest: the proposers alone keep it table-wise on one rank in the best
    plan they suggest; the refinement step may only improve the rating, and it is off when the caller chooses the proposers."""
    tables = [EmbeddingBagConfig(name=f"t{i}", embedding_dim=128, num_embeddings=4_000_000, feature_names=[f"f{i}"]) for i in range(10)]
    pooling = [1, 1, 1, 2, 3, 4, 6, 9, 27, 100]
    constraints = {f"t{i}": ParameterConstraints(pooling_factors=[float(p)]) for i, p in enumerate(pooling)}
    ratings = {}
    for steps in (0, 16):
        planner = EmbeddingShardingPlanner(topology=Topology(world_size=8, local_world_size=8, compute_device="cuda"), batch_size=8192,
                                           constraints=constraints, debug=False, refine_steps=steps)
        plan = planner.plan(_Model(tables), [EmbeddingBagCollectionSharder()])
        assert set(plan.plan["sparse"]) == {f"t{i}" for i in range(10)}
        ratings[steps] = planner._perf_model.rate(planner._best_plan)
    assert ratings[16] <= ratings[0]
    chosen = EmbeddingShardingPlanner(topology=Topology(world_size=8, local_world_size=8, compute_device="cuda"), batch_size=8192,
                                      proposer=GreedyProposer(), debug=False)
    assert chosen._refine_steps == 0


def test_stored_plan_is_reused_and_a_plan_for_other_inputs_is_refused():
    """A plan stored as {storage_hash: option} comes back as the same placement without a search; the loader's fingerprint of the
    planner inputs must match (cf. ``torchrec/distributed/planner/tests/test_planners.py`` plan-loader cases)."""
    import copy

    from torchrec_b200.distributed.planner.planners import EmbeddingPlannerBase, extract_plan
    from torchrec_b200.distributed.planner.types import PlanLoader

    sharders = [EmbeddingBagCollectionSharder()]
    first = EmbeddingShardingPlanner(topology=_topo(4), batch_size=256, debug=False)
    assert isinstance(first, EmbeddingPlannerBase)
    plan = first.plan(_Model(_tables(4)), sharders)
    stored = {o.storage_hash(): copy.deepcopy(o) for o in first._best_plan}
    assert len(stored) == 4

    class _Loader(PlanLoader):
        def __init__(self, options, fingerprint):
            self.options, self.fingerprint, self.loads = options, fingerprint, 0

        def load(self):
            self.loads += 1
            return self.options

        def plan_context_hash(self):
            return self.fingerprint

    loader = _Loader(stored, first.hash_planner_context_inputs_str())

    class _NeverProposer(GreedyProposer):
        def propose(self):
            raise AssertionError("a stored plan must skip the search")

    again = EmbeddingShardingPlanner(topology=_topo(4), batch_size=256, debug=False, proposer=_NeverProposer(), plan_loader=loader)
    replayed = again.plan(_Model(_tables(4)), sharders)
    assert loader.loads == 1
    for name, ps in plan.plan["sparse"].items():
        other = replayed.plan["sparse"][name]
        assert (ps.sharding_type, ps.compute_kernel, ps.ranks) == (other.sharding_type, other.compute_kernel, other.ranks)
        assert [(s.shard_sizes, s.shard_offsets) for s in ps.sharding_spec.shards] == [(s.shard_sizes, s.shard_offsets) for s in other.sharding_spec.shards]

    other_batch = EmbeddingShardingPlanner(topology=_topo(4), batch_size=512, debug=False, plan_loader=loader)
    with pytest.raises(PlannerError) as err:
        other_batch.plan(_Model(_tables(4)), sharders)
    assert err.value.error_type == PlannerErrorType.PLANNER_INPUT_CONTEXT_MISMATCH

    # a stored plan that lacks a table of the model cannot be used
    options = EmbeddingEnumerator(topology=_topo(4), batch_size=256).enumerate(_Model(_tables(4)), sharders)
    partial = dict(list(stored.items())[:3])
    with pytest.raises(PlannerError) as err:
        extract_plan(options, partial)
    assert err.value.error_type == PlannerErrorType.PLAN_LOADING_FAILED


def test_pipeline_io_cost_offload_stats_and_small_planner_helpers():
    from torchrec_b200.distributed.planner.partitioners import OrderedDeviceHardware
    from torchrec_b200.distributed.planner.shard_estimators import EmbeddingOffloadStats, calculate_pipeline_io_cost
    from torchrec_b200.distributed.planner.stats import round_to_one_sigfig
    from torchrec_b200.distributed.planner.types import DeviceHardware, Perf, Storage
    from torchrec_b200.distributed.sharding_plan import placement_helper
    from torchrec_b200.distributed.types import PipelineType

    assert calculate_pipeline_io_cost(100, 1000, 50, PipelineType.NONE, None) == 1100
    assert calculate_pipeline_io_cost(100, 1000, 50, PipelineType.TRAIN_SPARSE_DIST, None) == 200
    assert calculate_pipeline_io_cost(100, 1000, 50, PipelineType.TRAIN_SPARSE_DIST, None, count_ephemeral_storage_cost=True) == 1200
    assert calculate_pipeline_io_cost(100, 1000, 50, PipelineType.TRAIN_PREFETCH_SPARSE_DIST, None) == 300 + 350
    assert calculate_pipeline_io_cost(100, 1000, 50, PipelineType.TRAIN_PREFETCH_SPARSE_DIST, 6) == 300 + 100
    assert calculate_pipeline_io_cost(100, 1000, 50, PipelineType.TRAIN_SPARSE_DIST, None, is_inference=True) == 0

    # 10 bins over 100 rows; 60 % of the lookups reuse within 10 rows, 40 % within 50
    hist = torch.zeros(10)
    hist[0], hist[4] = 60.0, 40.0
    stats = EmbeddingOffloadStats(cacheability=0.3, expected_lookups=77, mrc_hist_counts=hist, height=100)
    assert stats.expected_lookups == 77 and stats.cacheability == 0.3
    assert abs(stats.expected_miss_rate(0.05) - 0.4) < 1e-6     # the first bin is reached: its 60 % hit
    assert abs(stats.expected_miss_rate(0.45) - 0.0) < 1e-6     # bin 4 reached: everything hits
    assert abs(stats.expected_miss_rate(0.3) - 0.4) < 1e-6
    assert stats.expected_miss_rate(0.0) == 1.0 and stats.expected_miss_rate(1.0) == 0.0
    assert float(EmbeddingOffloadStats.estimate_cache_miss_rate(torch.tensor(30.0), torch.zeros(4), torch.linspace(0, 100, 5))) == 0.0
    assert abs(EmbeddingOffloadStats.estimate_cacheability(hist) - (4 * 0.4) / 10) < 1e-6
    with pytest.raises(ValueError):
        EmbeddingOffloadStats(0.0, 0, torch.zeros(2, 2), 10)

    assert round_to_one_sigfig(0.0123) == "0.01" and round_to_one_sigfig(1234) == "1000" and round_to_one_sigfig(0.5) == "0.5"
    assert placement_helper("cuda", 3, 11) == "rank:11/cuda:3" and placement_helper("cpu", 3, 11) == "rank:0/cpu"

    # equally loaded devices: local rank 0 of host 1 (rank 4) comes before local rank 1 of host 0 (rank 1)
    mk = lambda rank, perf: OrderedDeviceHardware(DeviceHardware(rank=rank, storage=Storage(hbm=1, ddr=1), perf=Perf(fwd_compute=perf, fwd_comms=0, bwd_compute=0, bwd_comms=0)), 4)
    order = sorted([mk(1, 1.0), mk(4, 1.0), mk(0, 1.0), mk(5, 0.5)])
    assert [o.device.rank for o in order] == [5, 0, 4, 1]
