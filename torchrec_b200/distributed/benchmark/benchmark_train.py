"""Forward + backward time of a sharded ``EmbeddingBagCollection`` under each sharding type, and of the unsharded fused
single-device collection for comparison (``torchrec/distributed/benchmark/benchmark_train.py``).

    python -m torchrec_b200.distributed.benchmark.benchmark_train --num_tables 8
    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 2 -m torchrec_b200.distributed.benchmark.benchmark_train
"""
from __future__ import annotations

import argparse
import os
from typing import List

import torch
import torch.distributed as dist

from torchrec_b200.distributed import sharding_plan as sp
from torchrec_b200.distributed.benchmark.benchmark_base import BenchmarkResult, benchmark_func
from torchrec_b200.distributed.embeddingbag import EmbeddingBagCollectionSharder
from torchrec_b200.distributed.model_parallel import DistributedModelParallel
from torchrec_b200.distributed.types import ShardingEnv, ShardingPlan, ShardingType
from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward
from torchrec_b200.optim.rowwise_adagrad import RowWiseAdagrad
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


def make_inputs(keys: List[str], rows: int, batch: int, pooling: int, n: int, device: torch.device, seed: int) -> List[KeyedJaggedTensor]:
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        lengths = torch.randint(0, 2 * pooling + 1, (len(keys) * batch,), generator=g)
        values = torch.randint(0, rows, (int(lengths.sum()),), generator=g)
        out.append(KeyedJaggedTensor(keys=keys, values=values, lengths=lengths, stride=batch).to(device))
    return out


def benchmark_sharding(sharding_type: str, tables: List[EmbeddingBagConfig], inputs: List[KeyedJaggedTensor], device: torch.device, world: int, rank: int,
                       iters: int, warmup: int) -> BenchmarkResult:
    model = torch.nn.Module()
    model.ebc = EmbeddingBagCollection(tables=tables, device=torch.device("meta"))
    if sharding_type != ShardingType.DATA_PARALLEL.value:
        apply_optimizer_in_backward(RowWiseAdagrad, model.ebc.parameters(), {"lr": 0.01})
    gens = {ShardingType.TABLE_WISE.value: lambda i: sp.table_wise(rank=i % world), ShardingType.ROW_WISE.value: lambda i: sp.row_wise(),
            ShardingType.COLUMN_WISE.value: lambda i: sp.column_wise(ranks=[(i + j) % world for j in range(min(world, 2))]),
            ShardingType.DATA_PARALLEL.value: lambda i: sp.data_parallel(), ShardingType.TABLE_ROW_WISE.value: lambda i: sp.table_row_wise(host_index=0)}
    sharder = EmbeddingBagCollectionSharder()
    mplan = sp.construct_module_sharding_plan(model.ebc, {t.name: gens[sharding_type](i) for i, t in enumerate(tables)}, sharder=sharder, world_size=world,
                                              local_size=world, device_type=device.type)
    dmp = DistributedModelParallel(model, env=ShardingEnv.from_process_group(dist.group.WORLD), device=device, plan=ShardingPlan({"ebc": mplan}), sharders=[sharder])
    state = {"i": 0}

    def run_iter() -> None:
        kjt = inputs[state["i"] % len(inputs)]
        state["i"] += 1
        out = dmp.module.ebc(kjt).wait().values()
        out.backward(torch.ones_like(out))

    return benchmark_func(f"ebc-{sharding_type}", run_iter, num_iters=iters, warmup_iters=warmup, device=device, rank=rank)


def main() -> None:
    p = argparse.ArgumentParser()
    p.add_argument("--num_tables", type=int, default=8)
    p.add_argument("--rows", type=int, default=100_000)
    p.add_argument("--dim", type=int, default=128)
    p.add_argument("--batch_size", type=int, default=2048)
    p.add_argument("--pooling", type=int, default=10)
    p.add_argument("--iters", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--sharding_types", type=str, default="table_wise,row_wise,column_wise,data_parallel")
    a = p.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    use_cuda = torch.cuda.is_available()
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29562")
    dist.init_process_group("nccl" if use_cuda else "gloo", rank=rank, world_size=world)
    keys = [f"f{i}" for i in range(a.num_tables)]
    tables = [EmbeddingBagConfig(name=f"t{i}", embedding_dim=a.dim, num_embeddings=a.rows, feature_names=[k]) for i, k in enumerate(keys)]
    inputs = make_inputs(keys, a.rows, a.batch_size, a.pooling, 4, device, 100 + rank)
    for st in a.sharding_types.split(","):
        res = benchmark_sharding(st, tables, inputs, device, world, rank, a.iters, a.warmup)
        if rank == 0:
            print(res, flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
