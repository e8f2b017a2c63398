"""Sequence-recommender training throughput: BERT4Rec (2 bidirectional layers, 4 heads, hidden 256, FFN 1024) over an item table of
20M rows x dim 256 in bf16 held by a column-wise sharded ``EmbeddingCollection`` (unpooled lookups, jagged sequence all-to-all),
sequence lengths uniform in [20, 200], Zipf(1.1) item ids, 15% of the positions masked, sampled softmax over the target and 8192
uniform negatives, batch 4096 per rank, Adam lr 1e-3 (fused into the lookup's backward for the table).

    python -m torchrec_b200.distributed.benchmark.benchmark_sequence --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 -m torchrec_b200.distributed.benchmark.benchmark_sequence

One JSON line: sequences/s and tokens/s over all ranks, device-timed, max over ranks.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import socket

import torch
import torch.distributed as dist


def make_batch(batch_size: int, min_len: int, max_len: int, vocab: int, zipf_s: float, mask_prob: float, negatives: int, gen: torch.Generator):
    from torchrec_b200.models.bert4rec import BERT4RecSampled

    lengths = torch.randint(min_len, max_len + 1, (batch_size,), generator=gen)
    n = int(lengths.sum())
    # bounded Zipf(s) by inverse transform of the continuous envelope
    u = torch.rand(n, generator=gen, dtype=torch.float64)
    a = 1.0 - zipf_s
    ids = ((u * ((vocab - 1) ** a - 1.0) + 1.0) ** (1.0 / a)).long().clamp(1, vocab - 2)
    masked = torch.rand(n, generator=gen) < mask_prob
    inputs = torch.where(masked, torch.full_like(ids, vocab - 1), ids)
    offsets = torch.cat([torch.zeros(1, dtype=torch.long), lengths.cumsum(0)])
    row = torch.repeat_interleave(torch.arange(batch_size), lengths)
    col = torch.arange(n) - offsets[:-1][row]
    pos = (row * max_len + col)[masked]
    neg = torch.randint(1, vocab - 1, (negatives,), generator=gen)
    return BERT4RecSampled.make_input(inputs, lengths, ids[masked], neg), pos, n


def main() -> None:
    p = argparse.ArgumentParser()
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--batch-per-rank", type=int, default=4096)
    p.add_argument("--vocab", type=int, default=20_000_000)
    p.add_argument("--dim", type=int, default=256)
    p.add_argument("--min-len", type=int, default=20)
    p.add_argument("--max-len", type=int, default=200)
    p.add_argument("--negatives", type=int, default=8192)
    p.add_argument("--pool", type=int, default=4, help="distinct batches cycled")
    p.add_argument("--padded", action="store_true", help="run the encoder on padded [B, max_len, D] tensors through the library modules (the packed, fused path is the default)")
    p.add_argument("--library-loss", action="store_true", help="materialise the [P, 1 + N] scores and call the library's cross entropy on them")
    p.add_argument("--cpu", action="store_true", help="plumbing check on the host (gloo); not a benchmark")
    p.add_argument("--kernel-table", action="store_true", help="print the device time per kernel of one untimed step to stderr")
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
    from torchrec_b200.distributed.embedding import EmbeddingCollectionSharder
    from torchrec_b200.distributed.model_parallel import DistributedModelParallel
    from torchrec_b200.distributed.types import ShardingEnv, ShardingPlan
    from torchrec_b200.models.bert4rec import BERT4RecSampled
    from torchrec_b200.modules.embedding_configs import DataType
    from torchrec_b200.ops import _ext
    from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward
    from torchrec_b200.optim.keyed import CombinedOptimizer, KeyedOptimizerWrapper
    from torchrec_b200.optim.optimizers import in_backward_optimizer_filter

    if not a.cpu:
        _ext.require_cuda_ext("benchmark_sequence")
    torch.manual_seed(0)
    model = BERT4RecSampled(a.vocab, a.max_len, a.dim, nhead=4, num_layers=2, dim_feedforward=1024, dropout=0.1, device=device,
                            embedding_device=torch.device("meta"), data_type=DataType.BF16)
    model.packed = not a.padded
    if not a.cpu and not a.padded:
        from torchrec_b200.ops import dense_ops

        dense_ops.set_dense_compute_dtype(torch.bfloat16)  # the packed encoder's projections run on the tcgen05 GEMMs
    ec = model.history.ec
    apply_optimizer_in_backward(torch.optim.Adam, ec.parameters(), {"lr": 1e-3})
    sharder = EmbeddingCollectionSharder()
    n_col = min(world, a.dim // 32)
    mplan = sp.construct_module_sharding_plan(ec, {t: sp.column_wise(ranks=list(range(n_col))) for t in ("item_embedding", "item_output_embedding")}, sharder=sharder, world_size=world, local_size=world,
                                              device_type=device.type)
    dmp = DistributedModelParallel(model, env=ShardingEnv.from_process_group(dist.group.WORLD), device=device, plan=ShardingPlan({"history.ec": mplan}), sharders=[sharder])
    dense = KeyedOptimizerWrapper(dict(in_backward_optimizer_filter(dmp.named_parameters())), lambda ps: torch.optim.Adam(ps, lr=1e-3, foreach=True))
    opt = CombinedOptimizer([dmp.fused_optimizer, dense])
    gen = torch.Generator().manual_seed(100 + rank)
    batches, tokens = [], 0
    for _ in range(a.pool):
        kjt, pos, n = make_batch(a.batch_per_rank, a.min_len, a.max_len, a.vocab, 1.1, 0.15, a.negatives, gen)
        batches.append((kjt.to(device), pos.to(device)))
        tokens += n
    tokens_per_step = tokens / a.pool

    def step(i: int) -> torch.Tensor:
        kjt, pos = batches[i % len(batches)]
        opt.zero_grad()
        with torch.autocast(device.type, dtype=torch.bfloat16):
            if a.library_loss:
                logits = dmp(kjt, pos)
                loss = torch.nn.functional.cross_entropy(logits.float(), torch.zeros(logits.shape[0], dtype=torch.long, device=device))
            else:
                loss = dmp(kjt, pos, True)  # sampled-softmax cross entropy fused with its gradient
        loss.backward()
        opt.step()
        return loss

    for i in range(a.warmup):
        loss = step(i)
    dist.barrier()
    if a.cpu:
        import time

        t0 = time.perf_counter()
        for i in range(a.steps):
            loss = step(i)
        ms = torch.tensor([(time.perf_counter() - t0) * 1e3])
    else:
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(a.steps):
            loss = step(i)
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], device=device)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    tok = torch.tensor([tokens_per_step], device=device)
    dist.all_reduce(tok)
    ms_per_step = float(ms) / a.steps
    if a.kernel_table and rank == 0 and not a.cpu:
        import sys

        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            step(0)
            torch.cuda.synchronize()
        agg = {}
        for e in prof.events():
            if e.device_type == torch.autograd.DeviceType.CUDA:
                r = agg.setdefault(e.name[:100], [0.0, 0])
                r[0] += e.device_time_total
                r[1] += 1
        print(f"kernel table ({sum(v[0] for v in agg.values()) / 1e3:.2f} ms of device time):", file=sys.stderr)
        for name, (t, n) in sorted(agg.items(), key=lambda kv: -kv[1][0])[:30]:
            print(f"  {t / 1e3:8.3f} ms  x{n:<4d} {name}", file=sys.stderr)
    sharded_ec = next((m for m in dmp.modules() if hasattr(m, "_engine_state") and hasattr(m, "_need_indices")), None)
    exchange = "fused into the lookup over peer memory" if sharded_ec is not None and sharded_ec._engine_state == "on" else "library collectives"
    if rank == 0:
        print(json.dumps({
            "metric": "BERT4Rec train sequences/sec", "exchange": exchange, "encoder": "padded, library modules" if a.padded else "packed tokens, fused kernels", "value": a.batch_per_rank * world / (ms_per_step / 1e3), "unit": "sequences/s",
            "tokens_per_s": float(tok) / (ms_per_step / 1e3), "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms_per_step,
            "loss": float(loss.detach()), "higher_is_better": True, "scaling": "weak", "dtype": "bf16", "data": "synthetic (Zipf(1.1) items, lengths U[20,200], 15% masked)",
            "config": {"model": "BERT4Rec 2 layers, 4 heads, hidden 256, FFN 1024, sampled softmax 8192 negatives", "item_tables": f"input and output embeddings, each {a.vocab} x {a.dim} bf16",
                       "parallelism": f"column-wise x{n_col} EmbeddingCollection + dense DDP x{world}", "batch_per_rank": a.batch_per_rank,
                       "l2_policy": f"{a.pool} distinct batches cycled, two tables of {a.vocab * a.dim * 2 / 2**30:.1f} GiB"}}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
