"""Host-side micro-benchmark: transposing the per-key-per-rank strides of many received KJTs into their sharding contexts after the
input all-to-all.  This runs on the critical path of every variable-batch step, once per sharding group.

    python -m torchrec_b200.distributed.benchmark.benchmark_set_sharding_context_post_a2a --num_list 1000 --num_keys 100

Counterpart of ``torchrec/distributed/benchmark/benchmark_set_sharding_context_post_a2a.py:23-105``."""
from __future__ import annotations

import argparse
from typing import Callable, List

import torch

from torchrec_b200.distributed.benchmark.benchmark_base import BenchmarkResult, benchmark_func
from torchrec_b200.distributed.embedding_sharding import _set_sharding_context_post_a2a
from torchrec_b200.distributed.embedding import EmbeddingCollectionContext
from torchrec_b200.distributed.sharding.sequence_sharding import SequenceShardingContext
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


def _set_sharding_context_post_a2a_zip(kjts: List[KeyedJaggedTensor], ctx) -> None:
    """Same result through ``zip`` (one C-level transpose instead of nested indexing)."""
    for kjt, sharding_context in zip(kjts, getattr(ctx, "sharding_contexts", [])):
        if hasattr(sharding_context, "batch_size_per_rank_per_feature") and kjt.variable_stride_per_key() and kjt.stride_per_key_per_rank():
            sharding_context.batch_size_per_rank_per_feature = [list(col) for col in zip(*kjt.stride_per_key_per_rank())]


def op_bench(num_list: int, num_keys: int, func: Callable[..., None], num_iters: int = 10) -> BenchmarkResult:
    kjts = [KeyedJaggedTensor(keys=[f"k{i}" for i in range(num_keys)], values=torch.ones(num_keys, dtype=torch.int32), lengths=torch.ones(num_keys, dtype=torch.int32),
                              stride_per_key_per_rank=[[1]] * num_keys) for _ in range(num_list)]
    ctx = EmbeddingCollectionContext(sharding_contexts=[SequenceShardingContext(batch_size_per_rank_per_feature=[]) for _ in range(num_list)])
    res = benchmark_func(f"{func.__name__}-{num_list}-{num_keys}", lambda: func(kjts, ctx), num_iters=num_iters, warmup_iters=2, device=torch.device("cpu"), rank=0)
    print(res)
    return res


def main(argv=None) -> None:
    p = argparse.ArgumentParser(description=__doc__)
    p.add_argument("--num_list", type=int, default=100)
    p.add_argument("--num_keys", type=int, default=100)
    args = p.parse_args(argv)
    for func in (_set_sharding_context_post_a2a, _set_sharding_context_post_a2a_zip):
        op_bench(args.num_list, args.num_keys, func)


if __name__ == "__main__":
    main()
