"""Plan report: per-rank HBM / perf table, per-table shardings, imbalance statistics and the
critical-path estimate.  Counterpart of ``torchrec/distributed/planner/stats.py``.
"""
from __future__ import annotations

import logging
import math
from collections import defaultdict
from typing import Any, Dict, List, Optional, Tuple, Union, cast

from torch import nn

from torchrec_b200.distributed.planner.types import (
    Enumerator,
    ParameterConstraints,
    Perf,
    ShardingOption,
    Stats,
    Storage,
    StorageReservation,
    Topology,
)
from torchrec_b200.distributed.planner.utils import bytes_to_gb, bytes_to_mb
from torchrec_b200.distributed.types import ModuleSharder, ShardingPlan, ShardingType

logger: logging.Logger = logging.getLogger(__name__)

MIN_WIDTH = 90


def _normalize(p: List[float]) -> List[float]:
    s = sum(p)
    return [x / s if s > 0 else 1.0 / max(len(p), 1) for x in p]


def _total_variation(p: List[float]) -> float:
    k = len(p)
    return max(abs(pi - 1.0 / k) for pi in p) if k > 0 else 0.0


def _total_distance(p: List[float]) -> float:
    k = len(p)
    return sum(abs(pi - 1.0 / k) for pi in p) if k > 0 else 0.0


def _chi_divergence(p: List[float], alpha: float = 1.0) -> float:
    k = len(p)
    return sum(abs(pi * k - 1.0) ** alpha / k for pi in p) if k > 0 else 0.0


def _kl_divergence(p: List[float]) -> float:
    k = len(p)
    return sum(pi * math.log(k * pi) for pi in p if pi > 0) if k > 0 else 0.0


def _calc_max_chi_divergence(N: int, alpha: float = 1.0) -> float:
    return (1.0 / N) ** alpha * (N - 1.0) + ((N - 1.0) / N) ** alpha * N ** (alpha - 1) if N > 0 else 0.0


def _calc_max_kl_divergence(N: int) -> float:
    return math.log(N) if N > 0 else 0.0


def _collapse_consecutive_ranks(ranks: List[int]) -> List[str]:
    if len(ranks) > 1 and ranks == list(range(min(ranks), max(ranks) + 1)):
        return [f"{min(ranks)}-{max(ranks)}"]
    return [str(r) for r in ranks]


def _generate_rank_hbm_stats(per_rank_hbm: List[int], func) -> float:
    total = sum(per_rank_hbm)
    percentages = [h / total for h in per_rank_hbm] if total > 0 else [1.0 / max(len(per_rank_hbm), 1)] * len(per_rank_hbm)
    return func(percentages)


def _generate_max_text(perfs: List[float]) -> str:
    max_perf = max(perfs) if perfs else 0.0
    idx = [str(i) for i, p in enumerate(perfs) if p == max_perf]
    return f"{round(max_perf, 3)} ms on ranks {','.join(idx[:8])}{'...' if len(idx) > 8 else ''}"


def _reduce_int_list(ranks: List[int]) -> str:
    if not ranks:
        return ""
    out, start, prev = [], ranks[0], ranks[0]
    for r in ranks[1:]:
        if r == prev + 1:
            prev = r
            continue
        out.append(f"{start}-{prev}" if prev > start else str(start))
        start = prev = r
    out.append(f"{start}-{prev}" if prev > start else str(start))
    return ",".join(out)


class EmbeddingStats(Stats):
    """Logs a human-readable report of the chosen plan."""

    def __init__(self) -> None:
        self._width = MIN_WIDTH
        self._stats_table: List[str] = []

    def log(self, sharding_plan: ShardingPlan, topology: Topology, batch_size: int, storage_reservation: StorageReservation,
            num_proposals: int, num_plans: int, run_time: float, best_plan: List[ShardingOption],
            constraints: Optional[Dict[str, ParameterConstraints]] = None, sharders: Optional[List[ModuleSharder[nn.Module]]] = None,
            enumerator: Optional[Enumerator] = None, debug: bool = True) -> None:
        W = topology.world_size
        shard_by_fqn = {so.fqn: so for so in best_plan}
        used_hbm = [0] * W
        used_ddr = [0] * W
        perf: List[Perf] = [Perf(0, 0, 0, 0) for _ in range(W)]
        per_rank_types: List[Dict[str, int]] = [defaultdict(int) for _ in range(W)]
        table_rows: List[List[str]] = []
        for so in best_plan:
            ranks = sorted({cast(int, s.rank) for s in so.shards})
            for s in so.shards:
                r = cast(int, s.rank)
                used_hbm[r] += cast(Storage, s.storage).hbm
                used_ddr[r] += cast(Storage, s.storage).ddr
                perf[r] += cast(Perf, s.perf)
                per_rank_types[r][_abbr(so.sharding_type)] += 1
            table_rows.append([
                so.fqn, _abbr(so.sharding_type), so.compute_kernel, f"{so.total_perf:.3f}", f"{bytes_to_gb(so.total_storage.hbm):.3f}",
                str(list(so.tensor.shape)), ",".join(_collapse_consecutive_ranks(ranks)),
                ",".join(f"{p:g}" for p in so.input_lengths),
            ])
        reserved = storage_reservation.last_reserved_topology
        lines: List[str] = []
        lines.append("--- Planner Statistics ---")
        lines.append(f"--- Evaluated {num_proposals} proposal(s), found {num_plans} possible plan(s), ran for {run_time:.2f}s ---")
        lines.append(f"--- World size {W}, local world size {topology.local_world_size}, compute device {topology.compute_device}, batch size {batch_size} ---")
        header = ["Rank", "HBM (GB)", "DDR (GB)", "Perf (ms)", "fwd comp", "fwd comm", "bwd comp", "bwd comm", "Shardings"]
        rows = [header]
        for r in range(W):
            cap = topology.devices[r].storage
            hbm_pct = used_hbm[r] / cap.hbm if cap.hbm else 0.0
            rows.append([
                str(r), f"{bytes_to_gb(used_hbm[r]):.3f} ({hbm_pct:.0%})", f"{bytes_to_gb(used_ddr[r]):.3f}", f"{perf[r].total:.3f}",
                f"{perf[r].fwd_compute:.3f}", f"{perf[r].fwd_comms:.3f}", f"{perf[r].bwd_compute:.3f}", f"{perf[r].bwd_comms:.3f}",
                " ".join(f"{k}:{v}" for k, v in sorted(per_rank_types[r].items())),
            ])
        lines.extend(_format_table(rows))
        lines.append("")
        rows = [["FQN", "Sharding", "Kernel", "Perf (ms)", "HBM (GB)", "Shape", "Ranks", "Pooling"]] + table_rows
        lines.extend(_format_table(rows))
        totals = [p.total for p in perf]
        lines.append("")
        lines.append(f"Longest critical path (max over ranks): {_generate_max_text(totals)}")
        lines.append(f"Sum of per-rank maxima per direction: fwd {max(max(p.fwd_compute, p.fwd_comms) for p in perf):.3f} ms, bwd {max(max(p.bwd_compute, p.bwd_comms) for p in perf):.3f} ms")
        n = _normalize(totals)
        lines.append(f"Perf imbalance: total variation {_total_variation(n):.3f}, total distance {_total_distance(n):.3f}, chi {_chi_divergence(n):.3f}, KL {_kl_divergence(n):.3f}")
        nh = _normalize([float(h) for h in used_hbm])
        lines.append(f"HBM imbalance: total variation {_total_variation(nh):.3f}, total distance {_total_distance(nh):.3f}, chi {_chi_divergence(nh):.3f}, KL {_kl_divergence(nh):.3f}")
        lines.append(f"Peak HBM: {bytes_to_gb(max(used_hbm)):.3f} GB on rank {used_hbm.index(max(used_hbm))}; "
                     f"reserved per rank: {bytes_to_gb(topology.devices[0].storage.hbm - reserved.devices[0].storage.hbm) if reserved else 0:.3f} GB")
        self._stats_table = lines
        self._width = max(MIN_WIDTH, max(len(l) for l in lines) + 4)
        if debug:
            self.log_table()

    def log_table(self) -> None:
        border = "#" * self._width
        logger.info(border)
        for l in self._stats_table:
            logger.info(f"# {l: <{self._width - 4}} #")
        logger.info(border)

    def report(self) -> str:
        return "\n".join(self._stats_table)


def _abbr(sharding_type: str) -> str:
    return {
        ShardingType.DATA_PARALLEL.value: "DP", ShardingType.TABLE_WISE.value: "TW", ShardingType.COLUMN_WISE.value: "CW",
        ShardingType.ROW_WISE.value: "RW", ShardingType.TABLE_ROW_WISE.value: "TWRW", ShardingType.TABLE_COLUMN_WISE.value: "TWCW",
        ShardingType.GRID_SHARD.value: "GRID",
    }.get(sharding_type, sharding_type)


def round_to_one_sigfig(x: float) -> str:
    """``x`` rounded to one significant figure, printed without exponent noise (``0.0123`` -> ``"0.01"``, ``1234`` -> ``"1000"``)."""
    return f'{float(f"{x:.1g}"):g}'


def _format_table(rows: List[List[str]]) -> List[str]:
    widths = [max(len(r[i]) for r in rows) for i in range(len(rows[0]))]
    out = []
    for i, r in enumerate(rows):
        out.append("  ".join(c.ljust(w) for c, w in zip(r, widths)))
        if i == 0:
            out.append("  ".join("-" * w for w in widths))
    return out


class NoopEmbeddingStats(Stats):
    def log(self, *args: Any, **kwargs: Any) -> None:
        pass
