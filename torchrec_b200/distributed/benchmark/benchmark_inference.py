"""Inference benchmark of quantized embedding modules: pooled (``--module ebc``) or sequence (``--module ec``) collections, on one
device or placed table-wise over the local devices.

    python -m torchrec_b200.distributed.benchmark.benchmark_inference --module ebc --forms quant,quant_sharded --world_size 2

Counterpart of ``torchrec/distributed/benchmark/benchmark_inference.py:67-288``."""
from __future__ import annotations

import argparse
from typing import List

import torch

from torchrec_b200.distributed.benchmark.benchmark_base import BenchmarkResult
from torchrec_b200.distributed.benchmark.embedding_collection_wrappers import ModuleForm, benchmark_ebc_module, get_tables
from torchrec_b200.modules.embedding_configs import DataType

# (rows, dim) of a mid-sized ranking model: a few large tables and a tail of small ones
DEFAULT_TABLE_SIZES = [(40_000_000, 128), (4_000_000, 128), (1_000_000, 128), (1_000_000, 128)] + [(100_000, 128)] * 8 + [(1000, 128)] * 8


def _run(pooled: bool, args: argparse.Namespace) -> List[BenchmarkResult]:
    sizes = [(min(r, args.row_cap) if args.row_cap else r, d) for r, d in DEFAULT_TABLE_SIZES][: args.num_tables or None]
    tables = get_tables(sizes, is_pooled=pooled, data_type=DataType.INT8)
    device = torch.device(args.device)
    out = []
    for name in args.forms.split(","):
        res = benchmark_ebc_module(tables, ModuleForm(name), batch_size=args.batch_size, pooling=args.pooling, num_iters=args.iters, warmup_iters=args.warmup,
                                   device=device, world_size=args.world_size, profile_dir=args.profile)
        print(res)
        out.append(res)
    return out


def benchmark_qebc(args: argparse.Namespace) -> List[BenchmarkResult]:
    return _run(True, args)


def benchmark_qec(args: argparse.Namespace) -> List[BenchmarkResult]:
    return _run(False, args)


def main(argv=None) -> List[BenchmarkResult]:
    p = argparse.ArgumentParser(description=__doc__)
    p.add_argument("--module", default="ebc", choices=["ebc", "ec", "both"])
    p.add_argument("--forms", default="float,quant", help="comma list of float | quant | quant_sharded")
    p.add_argument("--batch_size", type=int, default=2048)
    p.add_argument("--pooling", type=int, default=10)
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--world_size", type=int, default=1)
    p.add_argument("--num_tables", type=int, default=0)
    p.add_argument("--row_cap", type=int, default=0, help="cap rows per table (smoke runs)")
    p.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    p.add_argument("--profile", default="")
    args = p.parse_args(argv)
    out: List[BenchmarkResult] = []
    if args.module in ("ebc", "both"):
        out += benchmark_qebc(args)
    if args.module in ("ec", "both"):
        out += benchmark_qec(args)
    return out


if __name__ == "__main__":
    main()
