"""Micro-benchmarks of the hand-written kernels at DLRM-DCNv2 shapes: the tcgen05 GEMMs (plain and fused
epilogues) against ``torch.matmul``/``F.linear`` and the table-batched embedding forward / sort / backward.

    python -m torchrec_b200.distributed.benchmark.benchmark_kernels --op all
    python -m torchrec_b200.distributed.benchmark.benchmark_kernels --op tbe_bwd --small   # profiler-sized case

Times are medians of CUDA-event timings with an L2 flush (a 256 MiB write) before every timed call.
Counterpart of the raw table-batched-embedding benchmark of the reference
(``torchrec/distributed/benchmark/benchmark_split_table_batched_embeddings.py``).
"""
from __future__ import annotations

import argparse
from typing import Callable, List

import torch

DLRM_ROWS = [40000000, 39060, 17295, 7424, 20265, 3, 7122, 1543, 63, 40000000, 3067956, 405282, 10, 2209, 11938, 155, 4, 976,
             14, 40000000, 40000000, 40000000, 590152, 12973, 108, 36]
DLRM_POOLING = [3, 2, 1, 2, 6, 1, 1, 1, 1, 7, 3, 8, 1, 6, 9, 5, 1, 1, 1, 12, 100, 27, 10, 3, 1, 1]


def timeit(fn: Callable[[], object], n: int = 10, warm: int = 3) -> float:
    """Median milliseconds of ``fn`` over ``n`` runs after ``warm`` warm-ups, L2 flushed before each run."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
    flush = torch.empty(256 * 1024 * 1024 // 4, device="cuda")
    for s, e in evs:
        flush.zero_()
        s.record()
        fn()
        e.record()
    torch.cuda.synchronize()
    ts = sorted(s.elapsed_time(e) for s, e in evs)
    return ts[len(ts) // 2]


def bench_gemm_nt(M: int, shapes: List[tuple], n: int, warm: int) -> None:
    ops = torch.ops.trb200
    for (N, K) in shapes:
        a = torch.randn(M, K, device="cuda").bfloat16()
        b = torch.randn(N, K, device="cuda").bfloat16()
        bias = torch.randn(N, device="cuda")
        t1 = timeit(lambda: ops.gemm_nt_bf16(a, b, bias, 1, False), n, warm)
        t2 = timeit(lambda: torch.relu(torch.nn.functional.linear(a, b, bias.bfloat16())), n, warm)
        t3 = timeit(lambda: torch.matmul(a, b.t()), n, warm)
        fl = 2 * M * N * K
        print(f"NT  M={M} N={N} K={K}: tcgen05+bias+relu {t1:.3f} ms ({fl / t1 / 1e9:.0f} TF) | torch linear+relu {t2:.3f} ms | "
              f"matmul only {t3:.3f} ms ({fl / t3 / 1e9:.0f} TF)", flush=True)


def bench_gemm_cross(M: int, D: int, R: int, n: int, warm: int) -> None:
    """The low-rank cross layer's second GEMM with its fused epilogue ``y = x0 * (v W^T + b) + xl``."""
    ops = torch.ops.trb200
    v = torch.randn(M, R, device="cuda").bfloat16()
    w = torch.randn(D, R, device="cuda").bfloat16()
    bias = torch.randn(D, device="cuda")
    x0 = torch.randn(M, D, device="cuda").bfloat16()
    xl = torch.randn(M, D, device="cuda").bfloat16()
    t1 = timeit(lambda: ops.gemm_nt_bf16_cross(v, w, bias, x0, xl), n, warm)
    t2 = timeit(lambda: x0 * torch.nn.functional.linear(v, w, bias.bfloat16()) + xl, n, warm)
    fl = 2 * M * D * R
    byt = 4 * M * D * 2
    print(f"CROSS M={M} N={D} K={R}: tcgen05 fused {t1:.3f} ms ({fl / t1 / 1e9:.0f} TF, {byt / t1 / 1e6:.0f} GB/s epilogue traffic) | "
          f"torch unfused {t2:.3f} ms", flush=True)


def bench_gemm_tn(M: int, shapes: List[tuple], n: int, warm: int) -> None:
    ops = torch.ops.trb200
    for (N, K) in shapes:
        a = torch.randn(M, N, device="cuda").bfloat16()
        b = torch.randn(M, K, device="cuda").bfloat16()
        t1 = timeit(lambda: ops.gemm_tn_bf16(a, b), n, warm)
        t3 = timeit(lambda: torch.matmul(a.t(), b), n, warm)
        fl = 2 * M * N * K
        print(f"TN  Mc={M} N={N} K={K}: tcgen05 {t1:.3f} ms ({fl / t1 / 1e9:.0f} TF) | torch {t3:.3f} ms ({fl / t3 / 1e9:.0f} TF)", flush=True)


def bench_tbe(B: int, row_cap: int, which: str, n: int, warm: int) -> None:
    from torchrec_b200.modules.embedding_configs import PoolingMode
    from torchrec_b200.ops.tbe import EmbOptimType, OptimizerArgs, TableBatchedEmbeddingBags

    rows = [min(r, row_cap) for r in DLRM_ROWS]
    m = TableBatchedEmbeddingBags(
        [(r, 128) for r in rows], pooling_mode=PoolingMode.SUM, output_dtype=torch.bfloat16,
        optimizer_args=OptimizerArgs(EmbOptimType.EXACT_ROWWISE_ADAGRAD, 0.005), device="cuda",
    )
    m.init_embedding_weights_uniform(-0.01, 0.01)
    g = torch.Generator(device="cuda").manual_seed(0)
    idx, lens = [], []
    for r, p in zip(rows, DLRM_POOLING):
        u = torch.rand(B * p, device="cuda", generator=g)
        ids = ((r ** u) - 1).long().clamp(0, r - 1)  # heavy-headed (Zipf-like) ids
        idx.append((ids * 2654435761) % r)
        lens.append(torch.full((B,), p, device="cuda", dtype=torch.int64))
    idx = torch.cat(idx).to(torch.int32)
    off = torch.cat([torch.zeros(1, device="cuda", dtype=torch.int64), torch.cat(lens).cumsum(0)]).to(torch.int32)
    N = idx.numel()
    print(f"TBE B={B} ids={N} rows<= {row_cap} weights {m.weights.numel() * 4 / 2**30:.1f} GiB", flush=True)
    if which in ("tbe_fwd", "tbe", "all"):
        with torch.no_grad():
            t = timeit(lambda: m(idx, off), n, warm)
        print(f"tbe fwd {t:.3f} ms  {N * 512 / t / 1e6:.0f} GB/s gathered", flush=True)
    if which in ("tbe_sort", "tbe", "all"):
        t = timeit(lambda: m.build_plan(idx, off, None, B), n, warm)
        print(f"tbe plan (linearize + radix sort) {t:.3f} ms", flush=True)
    if which in ("tbe_bwd", "tbe", "all"):
        grad = torch.randn(B, 26 * 128, device="cuda").bfloat16()
        plan = m.build_plan(idx, off, None, B)
        uniq = int(torch.unique(plan.keys).numel())
        t = timeit(lambda: m._backward_impl(grad, idx, off, None, B, plan), n, warm)
        byt = uniq * 128 * 4 * 2 + grad.numel() * 2
        print(f"tbe bwd apply {t:.3f} ms  unique rows {uniq}  minimum traffic {byt / 1e9:.2f} GB -> {byt / t / 1e6:.0f} GB/s", flush=True)
    m.check_error()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="all", choices=["all", "gemm_nt", "gemm_tn", "gemm_cross", "tbe", "tbe_fwd", "tbe_sort", "tbe_bwd"])
    ap.add_argument("--small", action="store_true", help="profiler-sized case: few launches, a few GB on the device")
    ap.add_argument("--batch", type=int, default=65536)
    ap.add_argument("--row-cap", type=int, default=4000000)
    args = ap.parse_args()
    from torchrec_b200.ops import _ext

    _ext.require_cuda_ext("benchmark_kernels")
    M = 16384 if args.small else args.batch
    n, warm = (2, 1) if args.small else (10, 3)
    row_cap = min(args.row_cap, 200000) if args.small else args.row_cap
    if args.op in ("all", "gemm_nt"):
        bench_gemm_nt(M, [(512, 3456), (3456, 512), (1024, 3456), (1024, 1024), (512, 1024), (256, 512), (128, 256)], n, warm)
    if args.op in ("all", "gemm_cross"):
        bench_gemm_cross(M, 3456, 512, n, warm)
    if args.op in ("all", "gemm_tn"):
        bench_gemm_tn(M, [(512, 3456), (3456, 512), (1024, 3456), (1024, 1024), (512, 1024), (256, 512)], n, warm)
    if args.op in ("all", "tbe", "tbe_fwd", "tbe_sort", "tbe_bwd"):
        bench_tbe(M, row_cap, args.op, n, warm)
    print("gemm status", int(torch.ops.trb200.gemm_error_status()), flush=True)


if __name__ == "__main__":
    main()
