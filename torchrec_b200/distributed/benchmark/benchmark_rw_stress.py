"""Row-wise sharding stress: an ``EmbeddingBagCollection`` of 64 tables x 10M rows x dim 256 in fp16 with a fixed pooling factor
of 20 (sum pooling, uniform ids), batch 16384 per rank; one step is forward + backward with the fused row-wise Adagrad.  Besides
the step time, the phases of the fused engine are device-timed inside real steps -- input distribution, lookup fused with the
reduce-scatter, finalize, gradient all-gather, backward -- and reported as achieved GB/s over NVLink per rank and as a fraction of
the measured peer-copy bandwidth; the same three exchanges are also timed as library collectives with the step's shapes.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 --master-port 29512 \\
        -m torchrec_b200.distributed.benchmark.benchmark_rw_stress --steps 10 --warmup 3
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import socket

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0  # measured peer-copy bandwidth per direction per GPU
HBM_GBS = 6556.8    # measured copy bandwidth of one GPU


def _time(fn, iters: int, device: torch.device) -> float:
    for _ in range(3):
        fn()
    dist.barrier()
    if device.type == "cpu":
        import time

        t0 = time.perf_counter()
        for _ in range(iters):
            fn()
        ms = torch.tensor([(time.perf_counter() - t0) * 1e3 / iters])
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / iters], device=device)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms)


def main() -> None:
    p = argparse.ArgumentParser()
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--tables", type=int, default=64)
    p.add_argument("--rows", type=int, default=10_000_000)
    p.add_argument("--dim", type=int, default=256)
    p.add_argument("--pooling", type=int, default=20)
    p.add_argument("--batch-per-rank", type=int, default=16384)
    p.add_argument("--cpu", action="store_true", help="plumbing check on the host (gloo); not a benchmark")
    p.add_argument("--qcomm", action="store_true", help="16-bit exchanges: fp16 partial rows forward, bf16 gradients backward (quantised-comms config); default fp32")
    p.add_argument("--no-library-collectives", action="store_true", help="skip timing the exchanges as library collectives")
    a = p.parse_args()
    rank, world, local_rank = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    device = torch.device("cpu") if a.cpu else torch.device(f"cuda:{local_rank}")
    if not a.cpu:
        torch.cuda.set_device(device)
    if "MASTER_ADDR" not in os.environ:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            os.environ["MASTER_PORT"] = str(s.getsockname()[1])
    os.environ.setdefault("LOCAL_WORLD_SIZE", str(world))
    if a.cpu:
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120))
    else:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device, timeout=datetime.timedelta(seconds=120))

    from torchrec_b200.distributed import sharding_plan as sp
    from torchrec_b200.distributed.embeddingbag import EmbeddingBagCollectionSharder
    from torchrec_b200.distributed.model_parallel import DistributedModelParallel
    from torchrec_b200.distributed.types import ShardingEnv, ShardingPlan
    from torchrec_b200.modules.embedding_configs import DataType, EmbeddingBagConfig
    from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
    from torchrec_b200.ops import _ext
    from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward
    from torchrec_b200.optim.rowwise_adagrad import RowWiseAdagrad
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    if not a.cpu:
        _ext.require_cuda_ext("benchmark_rw_stress")
    weight_bytes = a.tables * a.rows * a.dim * 2 / world
    free = torch.cuda.mem_get_info(device)[0] if not a.cpu else 1 << 60
    if weight_bytes * 1.1 > free:
        raise SystemExit(f"{weight_bytes / 2**30:.0f} GiB of table shards per rank do not fit in {free / 2**30:.0f} GiB: use more ranks")
    keys = [f"f{i}" for i in range(a.tables)]
    tables = [EmbeddingBagConfig(name=f"t{i}", embedding_dim=a.dim, num_embeddings=a.rows, feature_names=[k], data_type=DataType.FP16) for i, k in enumerate(keys)]
    ebc = EmbeddingBagCollection(tables=tables, device=torch.device("meta"))
    model = torch.nn.Module()
    model.ebc = ebc
    apply_optimizer_in_backward(RowWiseAdagrad, ebc.parameters(), {"lr": 0.01, "eps": 1e-8})
    registry = None
    if a.qcomm:
        from torchrec_b200.distributed.fbgemm_qcomm_codec import CommType, QCommsConfig, get_qcomm_codecs_registry

        registry = get_qcomm_codecs_registry(QCommsConfig(forward_precision=CommType.FP16, backward_precision=CommType.BF16))
    sharder = EmbeddingBagCollectionSharder(fused_params={"output_dtype": DataType.FP16}, qcomm_codecs_registry=registry)
    mplan = sp.construct_module_sharding_plan(ebc, {t.name: sp.row_wise() for t in tables}, sharder=sharder, world_size=world, local_size=world, device_type=device.type)
    dmp = DistributedModelParallel(model, env=ShardingEnv.from_process_group(dist.group.WORLD), device=device, plan=ShardingPlan({"ebc": mplan}), sharders=[sharder])
    sebc = dmp.module.ebc
    B = a.batch_per_rank
    gen = torch.Generator(device=device).manual_seed(10 + rank) if not a.cpu else torch.Generator().manual_seed(10 + rank)
    batches = []
    for _ in range(2):
        values = torch.randint(0, a.rows, (a.tables * B * a.pooling,), generator=gen, device=device, dtype=torch.int64)
        lengths = torch.full((a.tables * B,), a.pooling, dtype=torch.int32, device=device)
        batches.append(KeyedJaggedTensor(keys=keys, values=values, lengths=lengths, stride=B))

    def step(i: int) -> None:
        out = sebc(batches[i % 2]).wait()
        out.values().backward(torch.ones_like(out.values()))

    for i in range(a.warmup):
        step(i)
    step_ms = _time(lambda: step(0), a.steps, device)

    # ---- the fused engine's phases, device-timed inside real steps ----------------------------------------------------
    ids_per_rank = a.tables * B * a.pooling
    frac = (world - 1) / world
    phases = None
    engine = getattr(sebc, "_engine", None)
    if engine is not None:
        engine.timing = {}
        for i in range(a.steps):
            step(i)
        local = engine.timing_summary()
        engine.timing = None
        t = torch.tensor([local.get(k, 0.0) for k in ("input_dist", "lookup_push", "finalize", "grad_publish", "backward_update")], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = dict(zip(("input_dist", "lookup_push", "finalize", "grad_publish", "backward_update"), [float(x) for x in t]))
        esz = {torch.float16: 2, torch.bfloat16: 2, torch.float32: 4}
        # bytes that must cross NVLink per rank and step (what leaves this GPU)
        in_bytes = frac * (ids_per_rank * 8 + a.tables * B * 4)
        rs_bytes = frac * B * a.tables * a.dim * world * esz[engine.stage_dtype]      # a partial row to every other owner ... of every sample
        gp_bytes = frac * B * a.tables * a.dim * world * esz[engine.grad_dtype]       # the gradient block to every other owner
        gbs = lambda nbytes, t_ms: nbytes / (t_ms / 1e3) / 1e9 if t_ms > 0 else 0.0
        # HBM side of the lookup: every id reads one table row; the backward reads a gradient row and reads + writes the table row
        row_bytes = a.dim * 2
        fwd_hbm = ids_per_rank * row_bytes
        phases = {
            "input_dist (count + scatter over peer stores)": {"ms": ms["input_dist"], "nvlink_GBps": gbs(in_bytes, ms["input_dist"]),
                                                              "fraction_of_nvlink": gbs(in_bytes, ms["input_dist"]) / NVLINK_GBS},
            "lookup + reduce-scatter (rows pushed to the owners inside the lookup kernel, incl. waiting for the ids)": {
                "ms": ms["lookup_push"], "nvlink_GBps": gbs(rs_bytes, ms["lookup_push"]), "fraction_of_nvlink": gbs(rs_bytes, ms["lookup_push"]) / NVLINK_GBS,
                "hbm_GBps_gathered": gbs(fwd_hbm, ms["lookup_push"]), "roofline_ms": max(rs_bytes / (NVLINK_GBS * 1e6), fwd_hbm / (HBM_GBS * 1e6))},
            "finalize (sum of partial rows, cast)": {"ms": ms["finalize"]},
            "gradient all-gather (blocks pushed to the owners)": {"ms": ms["grad_publish"], "nvlink_GBps": gbs(gp_bytes, ms["grad_publish"]),
                                                                   "fraction_of_nvlink": gbs(gp_bytes, ms["grad_publish"]) / NVLINK_GBS},
            "backward + row-wise Adagrad (local slab)": {"ms": ms["backward_update"]},
        }

    # ---- the three exchanges as library collectives with the step's shapes, for comparison -------------------------------
    id_send = torch.empty(ids_per_rank, dtype=torch.int64, device=device)
    id_recv = torch.empty_like(id_send)
    len_send = torch.empty(a.tables * B * world, dtype=torch.int32, device=device)
    len_recv = torch.empty_like(len_send)

    def input_dist() -> None:
        dist.all_to_all_single(len_recv, len_send)
        dist.all_to_all_single(id_recv, id_send)

    lib = None
    if not a.no_library_collectives:
        t_in = _time(input_dist, 10, device)
        in_b = (id_send.numel() * 8 + len_send.numel() * 4) * frac
        pooled = torch.empty(B * world, a.tables * a.dim, dtype=torch.float16, device=device)
        rs_out = torch.empty(B, a.tables * a.dim, dtype=torch.float16, device=device)
        t_rs = _time(lambda: dist.reduce_scatter_tensor(rs_out, pooled), 10, device)
        rs_b = pooled.numel() * 2 * frac
        t_ag = _time(lambda: dist.all_gather_into_tensor(pooled, rs_out), 10, device)
        g = lambda nbytes, t_ms: nbytes / (t_ms / 1e3) / 1e9
        lib = {"input_dist_a2a": {"ms": t_in, "GBps_per_rank": g(in_b, t_in)}, "pooled_reduce_scatter": {"ms": t_rs, "GBps_per_rank": g(rs_b, t_rs)},
               "grad_all_gather": {"ms": t_ag, "GBps_per_rank": g(rs_b, t_ag)}, "sum_ms": t_in + t_rs + t_ag}
    if rank == 0:
        print(json.dumps({
            "metric": "row-wise EBC step (forward + backward, fused row-wise Adagrad)", "n_gpus": world, "ms_per_step": step_ms,
            "samples_per_s": B * world / (step_ms / 1e3), "lookups_per_s": ids_per_rank * world / (step_ms / 1e3),
            "path": "fused sparse engine over peer memory" if engine is not None else "library collectives",
            "engine_phases": phases, "library_collectives_same_shapes": lib,
            "config": {"tables": a.tables, "rows": a.rows, "dim": a.dim, "dtype": "fp16", "pooling": a.pooling, "batch_per_rank": B, "data": "synthetic uniform ids",
                       "exchange_precision": "fp16 forward / bf16 backward" if a.qcomm else "fp32",
                       "timing": "CUDA events, max over ranks; phase times are taken inside real steps and include waiting for peers"}}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
