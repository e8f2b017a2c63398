"""Operator benchmark of the table-batched embedding kernel alone: forward, or forward + fused backward/optimizer, over uniform
tables.

    python -m torchrec_b200.distributed.benchmark.benchmark_split_table_batched_embeddings --num_tables 8 --embedding_dim 128 --train true

Counterpart of ``torchrec/distributed/benchmark/benchmark_split_table_batched_embeddings.py:41-130``."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from torchrec_b200.distributed.benchmark.benchmark_base import BenchmarkResult, benchmark_func, cmd_conf


@dataclass
class TBEBenchConfig:
    num_tables: int = 8
    num_embeddings: int = 1_000_000
    embedding_dim: int = 128
    batch_size: int = 8192
    pooling: int = 10
    train: bool = True
    optimizer: str = "exact_row_wise_adagrad"
    num_iters: int = 20
    warmup_iters: int = 5
    device: str = ""
    profile: str = ""


def op_bench(cfg: TBEBenchConfig) -> BenchmarkResult:
    from torchrec_b200.ops.tbe import EmbOptimType, OptimizerArgs, TableBatchedEmbeddingBags

    device = torch.device(cfg.device or ("cuda" if torch.cuda.is_available() else "cpu"))
    tbe = TableBatchedEmbeddingBags([(cfg.num_embeddings, cfg.embedding_dim)] * cfg.num_tables,
                                    optimizer_args=OptimizerArgs(optimizer=EmbOptimType(cfg.optimizer), learning_rate=0.01), device=device)
    gen = torch.Generator().manual_seed(0)
    batches = []
    for _ in range(4):
        lengths = torch.randint(0, 2 * cfg.pooling + 1, (cfg.num_tables * cfg.batch_size,), generator=gen)
        offsets = torch.cat([lengths.new_zeros(1), lengths.cumsum(0)])
        batches.append((torch.randint(0, cfg.num_embeddings, (int(offsets[-1]),), generator=gen).to(device), offsets.to(device)))
    state = {"i": 0}

    def step() -> None:
        ids, offs = batches[state["i"] % len(batches)]
        state["i"] += 1
        if cfg.train:
            tbe(ids, offs).sum().backward()
        else:
            with torch.no_grad():
                tbe(ids, offs)

    res = benchmark_func(f"tbe-{'train' if cfg.train else 'fwd'}-T{cfg.num_tables}-D{cfg.embedding_dim}-B{cfg.batch_size}", step, num_iters=cfg.num_iters,
                         warmup_iters=cfg.warmup_iters, device=device, rank=0, profile_dir=cfg.profile)
    print(res)
    return res


@cmd_conf
def main(cfg: TBEBenchConfig) -> None:
    op_bench(cfg)


if __name__ == "__main__":
    main()
