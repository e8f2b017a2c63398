"""Per-shard perf and storage estimators.

Perf: for every shard, estimated wall time (ms) of the lookup kernels and of the bytes they put on
NVLink, per sharding type.  Storage: table weights + fused optimizer state + input/output buffers
(scaled by the pipeline depth) per shard.

Same role and structure as ``torchrec/distributed/planner/shard_estimators.py``
(``EmbeddingPerfEstimator`` ``:97-934``, ``EmbeddingStorageEstimator`` ``:940-1739``); the constants
model a B200 and the totals follow ``Perf.total`` (overlapped compute and comms).
"""
from __future__ import annotations

import logging
import math
from typing import Dict, List, Optional, Tuple, Type, cast

import torch
from torch import nn

from torchrec_b200.distributed.embedding_types import EmbeddingComputeKernel
from torchrec_b200.distributed.planner.constants import (
    BATCHED_COPY_PERF_FACTOR,
    BIGINT_DTYPE,
    DP_ELEMENTWISE_KERNELS_PERF_FACTOR,
    FULL_BLOCK_EMB_DIM,
    HALF_BLOCK_PENALTY,
    QUARTER_BLOCK_PENALTY,
    UVM_CACHING_RATIO,
    WEIGHTED_KERNEL_MULTIPLIER,
    kernel_bw_lookup,
)
from torchrec_b200.distributed.planner.types import (
    CollectiveType,
    GeneralizedCommsBandwidth,
    ParameterConstraints,
    Perf,
    PlannerError,
    ShardEstimator,
    ShardingOption,
    Storage,
    Topology,
)
from torchrec_b200.distributed.planner.utils import prod, sharder_name
from torchrec_b200.distributed.types import CacheStatistics, CommOp, ModuleSharder, PipelineType, ShardingType
from torchrec_b200.modules.embedding_configs import DATA_TYPE_NUM_BITS, DataType

logger: logging.Logger = logging.getLogger(__name__)


def _tensor_elem_bytes(t: torch.Tensor) -> float:
    return float(t.element_size())


def _extract_comm_data_type_size(sharder: Optional[ModuleSharder[nn.Module]], sharding_option: ShardingOption) -> Tuple[float, float, float, float]:
    """Bytes per element on the wire for (fwd a2a, bwd a2a, fwd reduce-scatter, bwd all-gather)."""
    elem = _tensor_elem_bytes(sharding_option.tensor)
    fwd_a2a = bwd_a2a = fwd_rs = bwd_rs = elem
    reg = getattr(sharder, "qcomm_codecs_registry", None) if sharder is not None else None
    if reg:
        a2a = reg.get(CommOp.POOLED_EMBEDDINGS_ALL_TO_ALL.name if sharding_option.is_pooled else CommOp.SEQUENCE_EMBEDDINGS_ALL_TO_ALL.name)
        if a2a is not None:
            fwd_a2a = torch.tensor([], dtype=a2a.forward.quantized_dtype).element_size()
            bwd_a2a = torch.tensor([], dtype=a2a.backward.quantized_dtype).element_size()
        rs = reg.get(CommOp.POOLED_EMBEDDINGS_REDUCE_SCATTER.name)
        if rs is not None:
            fwd_rs = torch.tensor([], dtype=rs.forward.quantized_dtype).element_size()
            bwd_rs = torch.tensor([], dtype=rs.backward.quantized_dtype).element_size()
    return float(fwd_a2a), float(bwd_a2a), float(fwd_rs), float(bwd_rs)


# True when the row-wise output dist is the fused lookup + push kernel that skips empty bags (see _get_rw_sharding_perf)
RW_SPARSE_REDUCE_SCATTER: bool = False


class EmbeddingPerfEstimator(ShardEstimator):
    """Wall-time estimate of every shard of every option (fills ``shard.perf``)."""

    def __init__(self, topology: Topology, constraints: Optional[Dict[str, ParameterConstraints]] = None, is_inference: bool = False) -> None:
        self._topology = topology
        self._constraints = constraints
        self._is_inference = is_inference

    def estimate(self, sharding_options: List[ShardingOption], sharder_map: Optional[Dict[str, ModuleSharder[nn.Module]]] = None) -> None:
        if not sharder_map:
            sharder_map = {}
        for so in sharding_options:
            sharder = sharder_map.get(sharder_name(type(so.module[1])), None)
            caching_ratio = so.cache_load_factor
            num_poolings = [1.0] * so.num_inputs
            batch_sizes = [so.batch_size] * so.num_inputs
            is_weighted = False
            if self._constraints and self._constraints.get(so.name):
                c = self._constraints[so.name]
                if c.num_poolings:
                    num_poolings = c.num_poolings
                if c.batch_sizes:
                    batch_sizes = c.batch_sizes
                is_weighted = c.is_weighted
            module = so.module[1]
            if getattr(module, "is_weighted", None) is not None and callable(module.is_weighted):
                try:
                    is_weighted = is_weighted or bool(module.is_weighted())
                except Exception:
                    pass
            assert len(so.input_lengths) == len(num_poolings), "Provided `pooling_factors` and `num_poolings` constraints must match in length"
            assert len(so.input_lengths) == len(batch_sizes), "Provided `pooling_factors` and `batch_sizes` constraints must match in length"
            table_elem = float(DATA_TYPE_NUM_BITS.get(_dtype_to_data_type(so.tensor.dtype), 32)) / 8
            fwd_a2a, bwd_a2a, fwd_rs, bwd_rs = _extract_comm_data_type_size(sharder, so)
            out_elem = fwd_a2a
            prefetch_pipeline = bool(so.cache_params.prefetch_pipeline) if so.cache_params and so.cache_params.prefetch_pipeline is not None else False
            shard_perfs = self.perf_func_emb_wall_time(
                shard_sizes=[s.size for s in so.shards], compute_kernel=so.compute_kernel, compute_device=self._topology.compute_device,
                sharding_type=so.sharding_type, batch_sizes=batch_sizes, world_size=self._topology.world_size,
                local_world_size=self._topology.local_world_size, input_lengths=so.input_lengths, input_data_type_size=BIGINT_DTYPE,
                table_data_type_size=table_elem, output_data_type_size=out_elem, fwd_a2a_comm_data_type_size=fwd_a2a,
                bwd_a2a_comm_data_type_size=bwd_a2a, fwd_sr_comm_data_type_size=fwd_rs, bwd_sr_comm_data_type_size=bwd_rs,
                num_poolings=num_poolings, hbm_mem_bw=self._topology.hbm_mem_bw, ddr_mem_bw=self._topology.ddr_mem_bw,
                hbm_to_ddr_mem_bw=self._topology.hbm_to_ddr_mem_bw, comms_bandwidths=self._topology.comms_bandwidths,
                bwd_compute_multiplier=self._topology.bwd_compute_multiplier,
                weighted_feature_bwd_compute_multiplier=self._topology.weighted_feature_bwd_compute_multiplier,
                is_pooled=so.is_pooled, is_weighted=is_weighted, caching_ratio=caching_ratio, is_inference=self._is_inference,
                prefetch_pipeline=prefetch_pipeline, uneven_sharding_perf_multiplier=self._topology.uneven_sharding_perf_multiplier,
            )
            for shard, perf in zip(so.shards, shard_perfs):
                shard.perf = perf

    @classmethod
    def perf_func_emb_wall_time(
        cls, shard_sizes: List[List[int]], compute_kernel: str, compute_device: str, sharding_type: str, batch_sizes: List[int],
        world_size: int, local_world_size: int, input_lengths: List[float], input_data_type_size: float, table_data_type_size: float,
        output_data_type_size: float, fwd_a2a_comm_data_type_size: float, bwd_a2a_comm_data_type_size: float,
        fwd_sr_comm_data_type_size: float, bwd_sr_comm_data_type_size: float, num_poolings: List[float], hbm_mem_bw: float,
        ddr_mem_bw: float, hbm_to_ddr_mem_bw: float, comms_bandwidths: GeneralizedCommsBandwidth, bwd_compute_multiplier: float,
        weighted_feature_bwd_compute_multiplier: float, is_pooled: bool, is_weighted: bool = False, caching_ratio: Optional[float] = None,
        is_inference: bool = False, prefetch_pipeline: bool = False, expected_cache_fetches: float = 0,
        uneven_sharding_perf_multiplier: float = 1.0,
    ) -> List[Perf]:
        device_bw = kernel_bw_lookup(compute_device, compute_kernel, hbm_mem_bw, ddr_mem_bw, hbm_to_ddr_mem_bw, caching_ratio, prefetch_pipeline)
        if device_bw is None:
            raise PlannerError(f"No kernel bandwidth exists for this combo of compute device: {compute_device}, compute kernel: {compute_kernel}")
        common = dict(
            batch_sizes=batch_sizes, world_size=world_size, local_world_size=local_world_size, input_lengths=input_lengths,
            input_data_type_size=input_data_type_size, table_data_type_size=table_data_type_size,
            num_poolings=num_poolings, device_bw=device_bw, comms_bandwidths=comms_bandwidths,
            bwd_compute_multiplier=bwd_compute_multiplier, weighted_feature_bwd_compute_multiplier=weighted_feature_bwd_compute_multiplier,
            is_pooled=is_pooled, is_weighted=is_weighted, is_inference=is_inference,
        )
        perfs: List[Perf] = []
        for hash_size, emb_dim in shard_sizes:
            if sharding_type in (ShardingType.TABLE_WISE.value, ShardingType.COLUMN_WISE.value, ShardingType.TABLE_COLUMN_WISE.value):
                p = cls._get_tw_sharding_perf(emb_dim=emb_dim, fwd_comm=fwd_a2a_comm_data_type_size, bwd_comm=bwd_a2a_comm_data_type_size, **common)
            elif sharding_type == ShardingType.ROW_WISE.value:
                p = cls._get_rw_sharding_perf(emb_dim=emb_dim, fwd_comm=fwd_sr_comm_data_type_size if is_pooled else fwd_a2a_comm_data_type_size,
                                              bwd_comm=bwd_sr_comm_data_type_size if is_pooled else bwd_a2a_comm_data_type_size, shards=world_size, **common)
            elif sharding_type in (ShardingType.TABLE_ROW_WISE.value, ShardingType.GRID_SHARD.value):
                p = cls._get_rw_sharding_perf(emb_dim=emb_dim, fwd_comm=fwd_sr_comm_data_type_size, bwd_comm=bwd_sr_comm_data_type_size,
                                              shards=local_world_size, hierarchical=True, fwd_a2a=fwd_a2a_comm_data_type_size,
                                              bwd_a2a=bwd_a2a_comm_data_type_size, **common)
            elif sharding_type == ShardingType.DATA_PARALLEL.value:
                p = cls._get_dp_sharding_perf(emb_dim=emb_dim, num_rows=hash_size, output_data_type_size=output_data_type_size, **common)
            else:
                raise ValueError(f"Unrecognized or unsupported sharding type provided: {sharding_type}")
            perfs.append(p)
        return perfs

    @staticmethod
    def _block_penalty(emb_dim: int) -> float:
        if emb_dim >= FULL_BLOCK_EMB_DIM:
            return 1.0
        return HALF_BLOCK_PENALTY if emb_dim >= 64 else QUARTER_BLOCK_PENALTY

    @classmethod
    def _get_tw_sharding_perf(cls, batch_sizes, world_size, local_world_size, input_lengths, emb_dim, input_data_type_size, table_data_type_size,
                              fwd_comm, bwd_comm, num_poolings, device_bw, comms_bandwidths, bwd_compute_multiplier,
                              weighted_feature_bwd_compute_multiplier, is_pooled, is_weighted=False, is_inference=False) -> Perf:
        """The owner looks up the whole global batch and sends ``(W-1)/W`` of the pooled rows away."""
        batch_inputs = sum(x * y * z for x, y, z in zip(input_lengths, num_poolings, batch_sizes))
        batch_outputs = sum(x * y for x, y in zip(num_poolings, batch_sizes)) if is_pooled else batch_inputs
        input_read = math.ceil(batch_inputs * world_size * input_data_type_size) * (2 if is_weighted else 1)
        lookup = batch_inputs * world_size * max(emb_dim, 32) * table_data_type_size
        fwd_out = batch_outputs * world_size * emb_dim * fwd_comm
        bwd_out = batch_outputs * world_size * emb_dim * bwd_comm
        comms_bw = comms_bandwidths.get_bw(world_size=world_size, local_world_size=local_world_size, collective_type=CollectiveType.ALL_TO_ALL)
        remote = (world_size - 1) / world_size if world_size > 1 else 0.0
        fwd_comms = fwd_out * remote / comms_bw
        fwd_compute = (input_read + lookup + fwd_out) * cls._block_penalty(emb_dim) / device_bw
        if is_inference:
            return Perf(fwd_compute=fwd_compute, fwd_comms=fwd_comms, bwd_compute=0, bwd_comms=0)
        bwd_comms = bwd_out * remote / comms_bw
        bwd_compute = fwd_compute * bwd_compute_multiplier
        if is_weighted:
            bwd_compute = bwd_compute * weighted_feature_bwd_compute_multiplier + fwd_compute * WEIGHTED_KERNEL_MULTIPLIER
        return Perf(fwd_compute=fwd_compute, fwd_comms=fwd_comms, bwd_compute=bwd_compute, bwd_comms=bwd_comms)

    @classmethod
    def _get_rw_sharding_perf(cls, batch_sizes, world_size, local_world_size, input_lengths, emb_dim, input_data_type_size, table_data_type_size,
                              fwd_comm, bwd_comm, num_poolings, device_bw, comms_bandwidths, bwd_compute_multiplier,
                              weighted_feature_bwd_compute_multiplier, is_pooled, shards, is_weighted=False, is_inference=False,
                              hierarchical=False, fwd_a2a=0.0, bwd_a2a=0.0) -> Perf:
        """Every shard looks up ``1/shards`` of the ids of the global batch and contributes a partial sum for every
        bag of the global batch.  The library reduce-scatter moves the dense ``[B_global, D]`` partials of every
        shard.  A lookup kernel that pushes only the bags it touched straight into the owner's buffer moves less: a
        bag of ``P`` ids touches at most ``min(P, shards)`` shards; ``RW_SPARSE_REDUCE_SCATTER`` selects that
        model."""
        batch_inputs = sum(x * y * z for x, y, z in zip(input_lengths, num_poolings, batch_sizes)) / shards
        if is_pooled:
            touched = 1.0
            if RW_SPARSE_REDUCE_SCATTER:
                touched = sum(min(1.0, x / shards) if x < shards else 1.0 for x in input_lengths) / max(len(input_lengths), 1)
            batch_outputs = sum(x * y for x, y in zip(num_poolings, batch_sizes)) * max(touched, 1.0 / shards)
        else:
            batch_outputs = batch_inputs
        input_read = math.ceil(batch_inputs * world_size * input_data_type_size) * (2 if is_weighted else 1)
        lookup = batch_inputs * world_size * max(emb_dim, 32) * table_data_type_size
        fwd_out = batch_outputs * world_size * emb_dim * fwd_comm
        bwd_out = batch_outputs * world_size * emb_dim * bwd_comm
        comms_bw = comms_bandwidths.get_bw(world_size=shards, local_world_size=local_world_size, collective_type=CollectiveType.REDUCE_SCATTER)
        remote = (shards - 1) / shards if shards > 1 else 0.0
        fwd_comms = fwd_out * remote / comms_bw
        if hierarchical and world_size > local_world_size:
            x_bw = comms_bandwidths.get_bw(world_size=world_size, local_world_size=local_world_size, collective_type=CollectiveType.ALL_TO_ALL)
            fwd_comms += batch_outputs * (world_size / local_world_size) * emb_dim * fwd_a2a / x_bw
        fwd_compute = (input_read + lookup + fwd_out) * cls._block_penalty(emb_dim) / device_bw
        if is_inference:
            return Perf(fwd_compute=fwd_compute, fwd_comms=fwd_comms, bwd_compute=0, bwd_comms=0)
        bwd_comms = bwd_out * remote / comms_bw
        if hierarchical and world_size > local_world_size:
            x_bw = comms_bandwidths.get_bw(world_size=world_size, local_world_size=local_world_size, collective_type=CollectiveType.ALL_TO_ALL)
            bwd_comms += batch_outputs * (world_size / local_world_size) * emb_dim * bwd_a2a / x_bw
        bwd_batched_copy = bwd_out * BATCHED_COPY_PERF_FACTOR / device_bw if not is_pooled else 0.0
        bwd_compute = fwd_compute * bwd_compute_multiplier
        if is_weighted:
            bwd_compute = bwd_compute * weighted_feature_bwd_compute_multiplier + fwd_compute * WEIGHTED_KERNEL_MULTIPLIER
        return Perf(fwd_compute=fwd_compute, fwd_comms=fwd_comms, bwd_compute=bwd_compute + bwd_batched_copy, bwd_comms=bwd_comms)

    @classmethod
    def _get_dp_sharding_perf(cls, batch_sizes, world_size, local_world_size, input_lengths, emb_dim, input_data_type_size, table_data_type_size,
                              num_poolings, device_bw, comms_bandwidths, bwd_compute_multiplier, weighted_feature_bwd_compute_multiplier,
                              is_pooled, num_rows, output_data_type_size, is_weighted=False, is_inference=False) -> Perf:
        """Local lookup of the local batch; the dense gradient of the whole table is all-reduced."""
        batch_inputs = sum(x * y * z for x, y, z in zip(input_lengths, num_poolings, batch_sizes))
        batch_outputs = sum(x * y for x, y in zip(num_poolings, batch_sizes)) if is_pooled else batch_inputs
        input_read = math.ceil(batch_inputs * input_data_type_size) * (2 if is_weighted else 1)
        lookup = batch_inputs * emb_dim * table_data_type_size
        out_write = batch_outputs * emb_dim * table_data_type_size
        table_size = num_rows * emb_dim * table_data_type_size
        fwd_compute = (input_read + lookup + out_write) / device_bw
        if is_inference:
            return Perf(fwd_compute=fwd_compute, fwd_comms=0, bwd_compute=0, bwd_comms=0)
        num_nodes = min(world_size / local_world_size, 2)
        ar_bw = comms_bandwidths.get_bw(world_size=world_size, local_world_size=local_world_size, collective_type=CollectiveType.ALL_REDUCE)
        all_reduce = table_size * (2 * num_nodes - 1) / num_nodes / ar_bw
        if world_size > 2 * local_world_size:
            all_reduce *= 2
        optimizer_kernels = table_size * DP_ELEMENTWISE_KERNELS_PERF_FACTOR / device_bw
        bwd_compute = fwd_compute * bwd_compute_multiplier
        if is_weighted:
            bwd_compute = bwd_compute * weighted_feature_bwd_compute_multiplier + fwd_compute * WEIGHTED_KERNEL_MULTIPLIER
        return Perf(fwd_compute=fwd_compute, fwd_comms=0, bwd_compute=bwd_compute + optimizer_kernels, bwd_comms=all_reduce)


def _dtype_to_data_type(dtype: torch.dtype) -> DataType:
    return {
        torch.float32: DataType.FP32, torch.float16: DataType.FP16, torch.bfloat16: DataType.BF16, torch.uint8: DataType.INT8,
        torch.int8: DataType.INT8, torch.quint4x2: DataType.INT4, torch.quint2x4: DataType.INT2,
    }.get(dtype, DataType.FP32)


class EmbeddingStorageEstimator(ShardEstimator):
    """HBM / DDR bytes of every shard (fills ``shard.storage``)."""

    def __init__(self, topology: Topology, constraints: Optional[Dict[str, ParameterConstraints]] = None,
                 pipeline_type: PipelineType = PipelineType.NONE, run_embedding_at_peak_memory: bool = False, is_inference: bool = False) -> None:
        self._topology = topology
        self._constraints = constraints
        self._pipeline_type = pipeline_type
        self._run_embedding_at_peak_memory = run_embedding_at_peak_memory
        self._is_inference = is_inference

    def estimate(self, sharding_options: List[ShardingOption], sharder_map: Optional[Dict[str, ModuleSharder[nn.Module]]] = None) -> None:
        if not sharder_map:
            assert not sharding_options, "sharder_map not provided for sharding_options"
            return
        for so in sharding_options:
            sharder = sharder_map[sharder_name(type(so.module[1]))]
            caching_ratio = so.cache_load_factor
            num_poolings = [1.0] * so.num_inputs
            batch_sizes = [so.batch_size] * so.num_inputs
            if self._constraints and self._constraints.get(so.name):
                c = self._constraints[so.name]
                if c.num_poolings:
                    num_poolings = c.num_poolings
                if c.batch_sizes:
                    batch_sizes = c.batch_sizes
            fused_params = getattr(sharder, "fused_params", None) or {}
            optimizer_class = None
            if hasattr(so.tensor, "_optimizer_classes") and so.tensor._optimizer_classes:
                optimizer_class = so.tensor._optimizer_classes[0]
            # the lookup's outputs live from forward to backward: they count toward the peak unless the caller says that the
            # embedding step does not run at the model's memory peak
            count_ephemeral = True
            mpp = getattr(so.cache_params, "multipass_prefetch_config", None) if so.cache_params else None
            shard_storages = calculate_shard_storages(
                sharder=sharder, sharding_type=so.sharding_type, tensor=so.tensor, compute_device=self._topology.compute_device,
                compute_kernel=so.compute_kernel, shard_sizes=[s.size for s in so.shards], batch_sizes=batch_sizes,
                world_size=self._topology.world_size, local_world_size=self._topology.local_world_size, input_lengths=so.input_lengths,
                num_poolings=num_poolings, caching_ratio=caching_ratio if caching_ratio else UVM_CACHING_RATIO, is_pooled=so.is_pooled,
                input_data_type_size=BIGINT_DTYPE, output_data_type_size=float(so.tensor.element_size()), pipeline_type=self._pipeline_type,
                multipass_prefetch_max_pass=getattr(mpp, "num_passes", None),
                count_ephemeral_storage_cost=count_ephemeral, is_inference=self._is_inference, optimizer_class=optimizer_class,
                fused_params=fused_params,
            )
            for shard, storage in zip(so.shards, shard_storages):
                shard.storage = storage


def calculate_pipeline_io_cost(input_size: int, output_size: int, prefetch_size: int, pipeline_type: PipelineType,
                               multipass_prefetch_max_pass: Optional[int], count_ephemeral_storage_cost: bool = False,
                               is_inference: bool = False) -> int:
    """Bytes of id / output buffers that a train pipeline keeps alive at its peak, given the bytes of ONE batch's ids (``input_size``),
    outputs (``output_size``) and prefetched rows (``prefetch_size``).  A sparse-dist pipeline holds the ids of two batches, the
    prefetch pipeline three plus the prefetch burst (smaller when the prefetch is split into passes); outputs count only when
    short-lived buffers are counted; no pipeline: one batch of each; inference: nothing beyond the step itself.
    Same accounting as ``torchrec/distributed/planner/shard_estimators.py:1087-1127``."""
    if is_inference:
        return 0
    outputs = output_size if count_ephemeral_storage_cost else 0
    if pipeline_type == PipelineType.TRAIN_SPARSE_DIST:
        return 2 * input_size + outputs
    if pipeline_type == PipelineType.TRAIN_PREFETCH_SPARSE_DIST:
        passes = multipass_prefetch_max_pass or 1
        return 3 * input_size + int((1 + 6 / passes) * prefetch_size) + outputs
    return input_size + output_size


class EmbeddingOffloadStats(CacheStatistics):
    """Cache statistics of a table served through a software cache, from a histogram of its LRU miss-ratio curve.

    ``mrc_hist_counts[i]`` is the number of lookups that hit if the cache holds at least ``(i + 1) / n`` of the table's ``height``
    rows and would miss with less (a histogram of LRU stack distances over ``n`` equal bins).  ``expected_miss_rate(clf)`` is then the
    share of lookups whose stack distance is not covered by a cache of ``clf * height`` rows.  ``cacheability`` is the area under
    the miss-ratio curve (0: a tiny cache serves everything, 1: nothing is ever reused); ``expected_lookups`` the expected number of
    distinct ids per global batch.  Counterpart of ``torchrec/distributed/planner/shard_estimators.py:1660-1774``."""

    def __init__(self, cacheability: float, expected_lookups: int, mrc_hist_counts: torch.Tensor, height: int) -> None:
        if mrc_hist_counts.dim() != 1:
            raise ValueError(f"expected 1d tensor, got {mrc_hist_counts.dim()}d")
        if mrc_hist_counts.numel() == 0:
            raise ValueError("expected non-empty tensor")
        self._cacheability = cacheability
        self._expected_lookups = expected_lookups
        self.height = height
        self.hist: torch.Tensor = mrc_hist_counts
        self.bins: torch.Tensor = torch.linspace(0, height, len(mrc_hist_counts) + 1)

    @property
    def expected_lookups(self) -> int:
        return self._expected_lookups

    @property
    def cacheability(self) -> float:
        return self._cacheability

    def expected_miss_rate(self, clf: float) -> float:
        return float(EmbeddingOffloadStats.estimate_cache_miss_rate(torch.tensor(clf * self.height), self.hist, self.bins))

    @staticmethod
    def estimate_cache_miss_rate(cache_sizes: torch.Tensor, hist: torch.Tensor, bins: torch.Tensor) -> torch.Tensor:
        """Miss ratio at each of ``cache_sizes`` (rows): 1 - (share of the histogram in the bins that a cache of that size covers
        completely or reaches into).  A cache of k rows serves stack distances up to k - 1."""
        total = hist.sum()
        if float(total) == 0:
            return torch.zeros_like(cache_sizes, dtype=torch.float32)  # never used: never missed
        miss_after_bin = 1 - hist.cumsum(0) / total  # miss ratio once the cache reaches bin i
        sizes = cache_sizes.to(bins.dtype)
        reached = torch.bucketize(sizes - 1, bins, right=True) - 1  # index of the bin that holds distance k - 1; -1: below the first edge
        beyond = reached >= hist.numel()
        out = miss_after_bin[reached.clamp(0, hist.numel() - 1)]
        out = torch.where(reached < 0, torch.ones_like(out), out)
        return torch.where(beyond, torch.zeros_like(out), out)

    @staticmethod
    def estimate_cacheability(hist: torch.Tensor) -> float:
        """Area under the miss-ratio curve of ``hist``, in [0, 1]."""
        total = hist.sum()
        if float(total) == 0:
            return 0.0
        return float((1 - hist.cumsum(0) / total).sum() / hist.numel())


def _optimizer_multiplier(optimizer_class: Optional[Type[torch.optim.Optimizer]], shape: torch.Size, fused_params: Dict) -> float:
    """Optimizer state bytes as a multiple of the weight bytes."""
    name = optimizer_class.__name__ if optimizer_class is not None else str(fused_params.get("optimizer", ""))
    lname = name.lower()
    if not lname or lname in ("none",):
        return 0.0
    if "sgd" in lname:
        return 0.0
    if "rowwise" in lname.replace("_", "") and "adagrad" in lname:
        return 1.0 / shape[-1]
    if "partial" in lname:
        return 1.0 + 1.0 / shape[-1]
    if "adagrad" in lname:
        return 1.0
    if "adam" in lname or "lamb" in lname:
        return 2.0
    return 1.0


def calculate_shard_storages(
    sharder, sharding_type: str, tensor: torch.Tensor, compute_device: str, compute_kernel: str, shard_sizes: List[List[int]],
    batch_sizes: List[int], world_size: int, local_world_size: int, input_lengths: List[float], num_poolings: List[float],
    caching_ratio: float, is_pooled: bool, input_data_type_size: float, output_data_type_size: float, pipeline_type: PipelineType = PipelineType.NONE,
    count_ephemeral_storage_cost: bool = False, is_inference: bool = False, optimizer_class=None, fused_params: Optional[Dict] = None,
    multipass_prefetch_max_pass: Optional[int] = None,
) -> List[Storage]:
    fused_params = fused_params or {}
    tensor_storage = sharder.storage_usage(tensor, compute_device, compute_kernel)
    hbm_storage = tensor_storage.get("hbm", 0)
    ddr_storage = tensor_storage.get("ddr", 0)
    table_cached = compute_kernel in {EmbeddingComputeKernel.FUSED_UVM_CACHING.value, EmbeddingComputeKernel.QUANT_UVM_CACHING.value}
    if table_cached:
        hbm_storage = round(ddr_storage * caching_ratio)
    tensor_numel = max(prod(tensor.shape), 1)
    opt_mult = 0.0 if is_inference or compute_kernel == EmbeddingComputeKernel.DENSE.value and False else _optimizer_multiplier(optimizer_class, tensor.shape, fused_params)
    # io buffers
    batch_inputs_total = sum(x * y * z for x, y, z in zip(input_lengths, num_poolings, batch_sizes))
    batch_outputs_total = sum(x * y for x, y in zip(num_poolings, batch_sizes)) if is_pooled else batch_inputs_total
    storages: List[Storage] = []
    for size in shard_sizes:
        frac = prod(size) / tensor_numel
        emb_dim = size[1]
        if sharding_type == ShardingType.DATA_PARALLEL.value:
            in_sz = batch_inputs_total * input_data_type_size
            out_sz = batch_outputs_total * emb_dim * output_data_type_size
        elif sharding_type in (ShardingType.ROW_WISE.value,):
            in_sz = batch_inputs_total / world_size * world_size * input_data_type_size
            out_sz = batch_outputs_total * world_size * emb_dim * output_data_type_size
        elif sharding_type in (ShardingType.TABLE_ROW_WISE.value, ShardingType.GRID_SHARD.value):
            in_sz = batch_inputs_total / local_world_size * world_size * input_data_type_size
            out_sz = batch_outputs_total * world_size * emb_dim * output_data_type_size
        else:
            in_sz = batch_inputs_total * world_size * input_data_type_size
            out_sz = batch_outputs_total * world_size * emb_dim * output_data_type_size
        io = calculate_pipeline_io_cost(
            input_size=math.ceil(in_sz), output_size=math.ceil(out_sz), prefetch_size=math.ceil(in_sz) if table_cached else 0,
            pipeline_type=pipeline_type, multipass_prefetch_max_pass=multipass_prefetch_max_pass,
            count_ephemeral_storage_cost=count_ephemeral_storage_cost, is_inference=is_inference)
        w_hbm = math.ceil(hbm_storage * frac)
        w_ddr = math.ceil(ddr_storage * frac)
        o_hbm = math.ceil(w_hbm * opt_mult)
        o_ddr = math.ceil(w_ddr * opt_mult)
        if compute_device == "cuda":
            storages.append(Storage(hbm=w_hbm + o_hbm + io, ddr=w_ddr + o_ddr))
        else:
            storages.append(Storage(hbm=w_hbm + o_hbm, ddr=w_ddr + o_ddr + io))
    return storages
