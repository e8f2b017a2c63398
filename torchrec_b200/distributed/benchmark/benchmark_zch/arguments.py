"""Command-line flags of the ZCH benchmark (``torchrec/distributed/benchmark/benchmark_zch/arguments.py``)."""
from __future__ import annotations

import argparse
from typing import List, Optional


def parse_args(argv: Optional[List[str]] = None) -> argparse.Namespace:
    p = argparse.ArgumentParser(description="managed-collision embedding benchmark on synthetic skewed ids")
    p.add_argument("--zch_method", default="mpzch", choices=["mpzch", "sort_zch", "none"], help="'none' folds ids with a plain modulo (the collision baseline)")
    p.add_argument("--num_tables", type=int, default=4)
    p.add_argument("--zch_size", type=int, default=20_000, help="rows per table")
    p.add_argument("--distinct_ids", type=int, default=15_000, help="distinct raw ids per feature in the stream")
    p.add_argument("--zipf_alpha", type=float, default=1.05, help="skew of the id popularity")
    p.add_argument("--input_hash_size", type=int, default=2 ** 50)
    p.add_argument("--embedding_dim", type=int, default=64)
    p.add_argument("--batch_size", type=int, default=4096)
    p.add_argument("--pooling", type=int, default=4)
    p.add_argument("--num_float_features", type=int, default=13)
    p.add_argument("--train_batches", type=int, default=50)
    p.add_argument("--eval_batches", type=int, default=10)
    p.add_argument("--warmup_batches", type=int, default=3)
    p.add_argument("--lr", type=float, default=0.05)
    p.add_argument("--mpzch_num_buckets", type=int, default=4)
    p.add_argument("--mpzch_max_probe", type=int, default=64)
    p.add_argument("--eviction_interval", type=int, default=1)
    p.add_argument("--device", default="")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--json", default="", help="write the result dictionary to this file")
    return p.parse_args(argv)
